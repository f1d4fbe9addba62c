#include "nvls.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#ifndef SYS_pidfd_open
#define SYS_pidfd_open 434
#endif
#ifndef SYS_pidfd_getfd
#define SYS_pidfd_getfd 438
#endif

namespace bagua {

namespace {

// ---- the CUDA runtime as a MulticastPlatform ------------------------------------------
bool cuda_select_device(int device) { return cudaSetDevice(device) == cudaSuccess && cudaFree(nullptr) == cudaSuccess; }
void* cuda_driver_entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult st;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void* cuda_scratch_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void cuda_scratch_free(void* p) { cudaFree(p); }
bool cuda_to_scratch(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream) == cudaSuccess;
}
bool cuda_from_scratch(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
         cudaStreamSynchronize(stream) == cudaSuccess;
}
bool cuda_clear(void* mapped, size_t bytes, cudaStream_t stream) {
  return cudaMemsetAsync(mapped, 0, bytes, stream) == cudaSuccess && cudaStreamSynchronize(stream) == cudaSuccess;
}
const MulticastPlatform kCudaPlatform = {cuda_select_device, cuda_driver_entry, cuda_scratch_alloc, cuda_scratch_free,
                                         cuda_to_scratch,    cuda_from_scratch, cuda_clear};
const MulticastPlatform* g_platform = &kCudaPlatform;

// Driver entry points, resolved through the runtime so that nothing links against libcuda.
struct Driver {
  // pointer types come from the driver header's own declarations
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;

  template <typename F>
  bool get(const char* name, F*& fn, std::string* why) {
    void* p = g_platform->driver_entry(name);
    if (!p) {
      *why = std::string("driver entry point ") + name + " is not available";
      return false;
    }
    fn = reinterpret_cast<F*>(p);
    return true;
  }
  bool load(std::string* why) {
    return get("cuDeviceGet", DeviceGet, why) && get("cuDeviceGetAttribute", DeviceGetAttribute, why) &&
           get("cuGetErrorString", GetErrorString, why) &&
           get("cuMemGetAllocationGranularity", MemGetAllocationGranularity, why) &&
           get("cuMemCreate", MemCreate, why) && get("cuMemRelease", MemRelease, why) &&
           get("cuMemExportToShareableHandle", MemExportToShareableHandle, why) &&
           get("cuMemImportFromShareableHandle", MemImportFromShareableHandle, why) &&
           get("cuMemAddressReserve", MemAddressReserve, why) && get("cuMemAddressFree", MemAddressFree, why) &&
           get("cuMemMap", MemMap, why) && get("cuMemUnmap", MemUnmap, why) &&
           get("cuMemSetAccess", MemSetAccess, why) && get("cuMulticastCreate", MulticastCreate, why) &&
           get("cuMulticastAddDevice", MulticastAddDevice, why) && get("cuMulticastBindMem", MulticastBindMem, why) &&
           get("cuMulticastUnbind", MulticastUnbind, why) &&
           get("cuMulticastGetGranularity", MulticastGetGranularity, why);
  }
};

struct Impl {
  Driver drv;
  CUdevice dev = 0;
  int rank = 0, nranks = 0;
  size_t bytes = 0;
  CUmemGenericAllocationHandle mc = 0;
  bool have_mc = false, bound = false;
  CUmemGenericAllocationHandle mem[kMulticastMaxRanks] = {};
  bool have_mem[kMulticastMaxRanks] = {};
  CUdeviceptr va[kMulticastMaxRanks] = {};
  bool reserved[kMulticastMaxRanks] = {}, mapped[kMulticastMaxRanks] = {};
  CUdeviceptr mc_va = 0;
  bool mc_reserved = false, mc_mapped = false;
  int fd_mem = -1, fd_mc = -1;  // exported descriptors, open until every peer has imported them
};

void close_fds(Impl& s) {
  if (s.fd_mem >= 0) close(s.fd_mem);
  if (s.fd_mc >= 0) close(s.fd_mc);
  s.fd_mem = s.fd_mc = -1;
}

void teardown(Impl& s) {
  Driver& d = s.drv;
  close_fds(s);
  if (s.mc_mapped) d.MemUnmap(s.mc_va, s.bytes);
  if (s.mc_reserved) d.MemAddressFree(s.mc_va, s.bytes);
  if (s.bound) d.MulticastUnbind(s.mc, s.dev, 0, s.bytes);
  for (int p = 0; p < s.nranks; ++p) {
    if (s.mapped[p]) d.MemUnmap(s.va[p], s.bytes);
    if (s.reserved[p]) d.MemAddressFree(s.va[p], s.bytes);
    if (s.have_mem[p]) d.MemRelease(s.mem[p]);
  }
  if (s.have_mc) d.MemRelease(s.mc);
  s.mc_mapped = s.mc_reserved = s.bound = s.have_mc = false;
  for (int p = 0; p < kMulticastMaxRanks; ++p) s.mapped[p] = s.reserved[p] = s.have_mem[p] = false;
}

// Slabs that are still bound, so that a process can drop its multicast bindings before it
// exits even when the owning communicator is never destroyed.
std::mutex g_live_mu;
std::vector<Impl*> g_live;

// One record per rank, all-gathered after every step.
struct Note {
  int32_t ok;
  int32_t pid;
  int32_t fd_mem;
  int32_t fd_mc;
  uint64_t bytes;
};

// All-gathers `mine` through device buffers on the transport (the same way the arena trades its IPC handles).
bool gather_notes(Transport& t, int rank, int nranks, cudaStream_t stream, const Note& mine, std::vector<Note>* all) {
  const MulticastPlatform& pf = *g_platform;
  void* dev = pf.scratch_alloc(sizeof(Note) * (size_t)nranks);
  if (!dev) return false;
  all->assign((size_t)nranks, Note{});
  bool ok = pf.to_scratch((char*)dev + sizeof(Note) * (size_t)rank, &mine, sizeof(Note), stream);
  if (ok) {
    t.allgather((char*)dev + sizeof(Note) * (size_t)rank, dev, (int64_t)sizeof(Note), DType::U8);
    ok = pf.from_scratch(all->data(), dev, sizeof(Note) * (size_t)nranks, stream);
  }
  pf.scratch_free(dev);
  return ok;
}

// Duplicates descriptor `fd` of process `pid` into this process.
int steal_fd(int pid, int fd) {
  const int pidfd = (int)syscall(SYS_pidfd_open, pid, 0);
  if (pidfd < 0) return -1;
  const int got = (int)syscall(SYS_pidfd_getfd, pidfd, fd, 0);
  close(pidfd);
  return got;
}

}  // namespace

void set_multicast_platform(const MulticastPlatform* platform) { g_platform = platform ? platform : &kCudaPlatform; }

bool create_multicast_slab(Transport& transport, int rank, int nranks, int device, cudaStream_t stream, size_t bytes,
                           MulticastSlab* out, std::string* why) {
  *out = MulticastSlab{};
  if (nranks < 2 || nranks > kMulticastMaxRanks) {
    *why = "multicast slabs need 2.." + std::to_string(kMulticastMaxRanks) + " ranks";
    return false;
  }
  auto impl = std::make_unique<Impl>();
  Impl& s = *impl;
  Driver& d = s.drv;
  s.rank = rank;
  s.nranks = nranks;
  std::string local_why;
  std::vector<Note> notes;

  // Every step: do the local work, then trade {ok, ...}; the first rank that failed decides for all.
  auto agree = [&](bool ok, const char* step, Note mine = Note{}) -> bool {
    mine.ok = ok ? 1 : 0;
    if (!gather_notes(transport, rank, nranks, stream, mine, &notes)) {
      *why = std::string(step) + ": exchanging the result between ranks failed";
      teardown(s);
      return false;
    }
    for (int p = 0; p < nranks; ++p)
      if (!notes[p].ok) {
        *why = std::string(step) + " failed on rank " + std::to_string(p) + (p == rank ? ": " + local_why : std::string());
        teardown(s);
        return false;
      }
    return true;
  };
  auto check = [&](CUresult r, const char* what) -> bool {
    if (r == CUDA_SUCCESS) return true;
    const char* msg = nullptr;
    if (d.GetErrorString) d.GetErrorString(r, &msg);
    local_why = std::string(what) + ": " + (msg ? msg : "unknown driver error");
    return false;
  };

  // 1. capability
  bool ok = g_platform->select_device(device);
  if (!ok) local_why = "the device cannot be selected";
  ok = ok && d.load(&local_why);
  if (ok) ok = check(d.DeviceGet(&s.dev, device), "cuDeviceGet");
  if (ok) {
    int mc = 0, fd = 0;
    ok = check(d.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, s.dev), "query multicast support") &&
         check(d.DeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, s.dev),
               "query descriptor export support");
    if (ok && (!mc || !fd)) {
      ok = false;
      local_why = mc ? "memory cannot be exported as a file descriptor" : "the device does not support multicast";
    }
  }
  if (!agree(ok, "capability check")) return false;

  // 2. size
  CUmulticastObjectProp mprop;
  std::memset(&mprop, 0, sizeof(mprop));
  mprop.numDevices = (unsigned)nranks;
  mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAllocationProp aprop;
  std::memset(&aprop, 0, sizeof(aprop));
  aprop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  aprop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  aprop.location.id = device;
  aprop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran_mc = 0, gran_mem = 0;
  mprop.size = align_up(bytes, (size_t)2 << 20);
  ok = check(d.MulticastGetGranularity(&gran_mc, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED), "multicast granularity") &&
       check(d.MemGetAllocationGranularity(&gran_mem, &aprop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
             "allocation granularity");
  size_t gran = 0;
  if (ok) {
    gran = std::max(gran_mc, gran_mem);
    ok = gran > 0 && (gran % gran_mc == 0) && (gran % gran_mem == 0);
    if (!ok) local_why = "multicast and allocation granularities do not nest";
  }
  if (ok) {
    s.bytes = align_up(bytes, gran);
    mprop.size = s.bytes;
  }
  {
    Note n{};
    n.bytes = s.bytes;
    if (!agree(ok, "granularity query", n)) return false;
    for (int p = 0; p < nranks; ++p)
      if (notes[p].bytes != s.bytes) {
        *why = "ranks disagree on the slab size";
        teardown(s);
        return false;
      }
  }

  // 3. create: rank 0 the multicast object, every rank its memory; export both as descriptors
  if (rank == 0) {
    ok = check(d.MulticastCreate(&s.mc, &mprop), "cuMulticastCreate");
    s.have_mc = ok;
    if (ok)
      ok = check(d.MemExportToShareableHandle(&s.fd_mc, s.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                 "export the multicast object");
  }
  if (ok) {
    ok = check(d.MemCreate(&s.mem[rank], s.bytes, &aprop, 0), "cuMemCreate");
    s.have_mem[rank] = ok;
  }
  if (ok)
    ok = check(d.MemExportToShareableHandle(&s.fd_mem, s.mem[rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
               "export the memory");
  {
    Note n{};
    n.pid = (int32_t)getpid();
    n.fd_mem = s.fd_mem;
    n.fd_mc = s.fd_mc;
    if (!agree(ok, "allocation", n)) return false;
  }
  const std::vector<Note> owners = notes;

  // 4. import the peers' memory and, except on rank 0, the multicast object
  for (int p = 0; p < nranks && ok; ++p) {
    if (p == rank) continue;
    const int fd = steal_fd(owners[p].pid, owners[p].fd_mem);
    if (fd < 0) {
      ok = false;
      local_why = "pidfd_getfd on a peer's memory descriptor failed (errno " + std::to_string(errno) + ")";
      break;
    }
    ok = check(d.MemImportFromShareableHandle(&s.mem[p], (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
               "import a peer's memory");
    s.have_mem[p] = ok;
    close(fd);
  }
  if (ok && rank != 0) {
    const int fd = steal_fd(owners[0].pid, owners[0].fd_mc);
    if (fd < 0) {
      ok = false;
      local_why = "pidfd_getfd on the multicast descriptor failed (errno " + std::to_string(errno) + ")";
    } else {
      ok = check(d.MemImportFromShareableHandle(&s.mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                 "import the multicast object");
      s.have_mc = ok;
      close(fd);
    }
  }
  if (!agree(ok, "import")) return false;
  close_fds(s);  // every peer holds its own reference now

  // 5. join the multicast team; all devices must have joined before anyone binds
  ok = check(d.MulticastAddDevice(s.mc, s.dev), "cuMulticastAddDevice");
  if (!agree(ok, "joining the multicast team")) return false;

  // 6. bind this rank's memory at offset 0
  ok = check(d.MulticastBindMem(s.mc, 0, s.mem[rank], 0, s.bytes, 0), "cuMulticastBindMem");
  s.bound = ok;
  if (!agree(ok, "binding memory to the multicast object")) return false;

  // 7. map everything
  CUmemAccessDesc access;
  std::memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int p = 0; p < nranks && ok; ++p) {
    ok = check(d.MemAddressReserve(&s.va[p], s.bytes, gran, 0, 0), "reserve an address range");
    s.reserved[p] = ok;
    if (ok) {
      ok = check(d.MemMap(s.va[p], s.bytes, 0, s.mem[p], 0), "map memory");
      s.mapped[p] = ok;
    }
    if (ok) ok = check(d.MemSetAccess(s.va[p], s.bytes, &access, 1), "enable access to memory");
  }
  if (ok) {
    ok = check(d.MemAddressReserve(&s.mc_va, s.bytes, gran, 0, 0), "reserve the multicast address range");
    s.mc_reserved = ok;
  }
  if (ok) {
    ok = check(d.MemMap(s.mc_va, s.bytes, 0, s.mc, 0), "map the multicast object");
    s.mc_mapped = ok;
  }
  if (ok) ok = check(d.MemSetAccess(s.mc_va, s.bytes, &access, 1), "enable access to the multicast mapping");
  if (ok) {
    ok = g_platform->clear((void*)(uintptr_t)s.va[rank], s.bytes, stream);
    if (!ok) local_why = "clearing the slab failed";
  }
  if (!agree(ok, "mapping")) return false;

  for (int p = 0; p < nranks; ++p) out->base[p] = (char*)(uintptr_t)s.va[p];
  out->mc_base = (char*)(uintptr_t)s.mc_va;
  out->bytes = s.bytes;
  out->impl = impl.release();
  {
    std::lock_guard<std::mutex> g(g_live_mu);
    g_live.push_back(static_cast<Impl*>(out->impl));
  }
  return true;
}

void destroy_multicast_slab(MulticastSlab& slab) {
  if (!slab.impl) return;
  Impl* s = static_cast<Impl*>(slab.impl);
  {
    std::lock_guard<std::mutex> g(g_live_mu);
    for (size_t i = 0; i < g_live.size(); ++i)
      if (g_live[i] == s) {
        g_live.erase(g_live.begin() + (long)i);
        break;
      }
  }
  teardown(*s);  // a no-op for what release_all_multicast_slabs() already dropped
  delete s;
  slab = MulticastSlab{};
}

int release_all_multicast_slabs() {
  std::lock_guard<std::mutex> g(g_live_mu);
  int n = 0;
  for (Impl* s : g_live) {
    teardown(*s);
    ++n;
  }
  g_live.clear();
  return n;
}

}  // namespace bagua
