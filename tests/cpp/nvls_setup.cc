// The set-up of a multicast-mapped symmetric slab (csrc/comm/nvls.cc) on a machine without a
// GPU: N ranks run as threads of this process, the transport is an all-gather between threads,
// and the CUDA runtime and driver are replaced (set_multicast_platform) by a stand-in that hands
// out counted handles, real file descriptors and made-up addresses.  Checked:
//   * with a healthy stand-in every rank gets the slab, with the same size, distinct mappings of
//     every rank's memory and a multicast mapping;
//   * when any one driver call fails on any one rank, EVERY rank returns false and names the
//     same step (a rank that went on alone would later wait for peers that fell back), and
//     everything created up to then has been released again;
//   * release_all_multicast_slabs() followed by destroy_multicast_slab() releases everything
//     exactly once;
//   * no file descriptor is left open in any of these cases.
#include <cuda.h>
#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <barrier>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "comm/nvls.h"

using namespace bagua;

namespace {

// ---- transport between threads -------------------------------------------------------
struct Hub {
  explicit Hub(int n) : n(n), bar(n), slots((size_t)n) {}
  int n;
  std::barrier<> bar;
  std::vector<std::vector<char>> slots;
};

class ThreadTransport : public Transport {
 public:
  ThreadTransport(Hub& hub, int rank) : hub_(hub), rank_(rank) {}
  int rank() const override { return rank_; }
  int nranks() const override { return hub_.n; }
  const char* kind() const override { return "threads"; }
  void allgather(const void* send, void* recv, int64_t count, DType) override {
    hub_.slots[(size_t)rank_].assign((const char*)send, (const char*)send + count);
    hub_.bar.arrive_and_wait();
    for (int p = 0; p < hub_.n; ++p) std::memcpy((char*)recv + (size_t)p * (size_t)count, hub_.slots[(size_t)p].data(), (size_t)count);
    hub_.bar.arrive_and_wait();
  }
  void barrier() override { hub_.bar.arrive_and_wait(); }
  void allreduce(const void*, void*, int64_t, DType, ReductionOp) override { std::abort(); }
  void broadcast(void*, int64_t, DType, int) override { std::abort(); }
  void reduce(const void*, void*, int64_t, DType, int, ReductionOp) override { std::abort(); }
  void send(const void*, int64_t, DType, int) override { std::abort(); }
  void recv(void*, int64_t, DType, int) override { std::abort(); }
  void alltoall(const void*, void*, int64_t, DType) override { std::abort(); }
  void alltoall_v(const void*, const std::vector<int64_t>&, const std::vector<int64_t>&, void*, const std::vector<int64_t>&,
                  const std::vector<int64_t>&, DType) override {
    std::abort();
  }
  void gather(const void*, void*, int64_t, DType, int) override { std::abort(); }
  void scatter(const void*, void*, int64_t, DType, int) override { std::abort(); }
  void reduce_scatter(const void*, void*, int64_t, DType, ReductionOp) override { std::abort(); }
  void group_start() override {}
  void group_end() override {}
  void abort() override {}

 private:
  Hub& hub_;
  int rank_;
};

// ---- stand-in driver -------------------------------------------------------------------
thread_local int t_rank = -1;

struct Fake {
  std::mutex mu;
  std::string fail_call;  // name of the driver call that fails ...
  int fail_rank = -1;     // ... on this rank (-1: nowhere)
  bool multicast_supported = true;
  // live objects
  std::map<unsigned long long, int> handles;  // handle -> references held by ranks (create or import)
  unsigned long long next_handle = 100;
  std::map<unsigned long long, size_t> reserved;  // address -> bytes
  std::map<unsigned long long, int> mapped;       // address -> 1
  int bound = 0;
  unsigned long long next_va = 0x7000000000ull;
  int calls = 0;
  bool fails_here(const char* name) {
    ++calls;
    return fail_rank == t_rank && fail_call == name;
  }
} g_fake;

#define FAKE_ENTER(name)                        \
  std::lock_guard<std::mutex> guard(g_fake.mu); \
  if (g_fake.fails_here(name)) return CUDA_ERROR_NOT_SUPPORTED

CUresult fk_DeviceGet(CUdevice* dev, int ordinal) {
  FAKE_ENTER("cuDeviceGet");
  *dev = ordinal;
  return CUDA_SUCCESS;
}
CUresult fk_DeviceGetAttribute(int* v, CUdevice_attribute attr, CUdevice) {
  FAKE_ENTER("cuDeviceGetAttribute");
  *v = attr == CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED ? (g_fake.multicast_supported ? 1 : 0) : 1;
  return CUDA_SUCCESS;
}
CUresult fk_GetErrorString(CUresult, const char** s) {
  *s = "injected failure";
  return CUDA_SUCCESS;
}
CUresult fk_MemGetAllocationGranularity(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) {
  FAKE_ENTER("cuMemGetAllocationGranularity");
  *g = (size_t)2 << 20;
  return CUDA_SUCCESS;
}
CUresult fk_MulticastGetGranularity(size_t* g, const CUmulticastObjectProp*, CUmulticastGranularity_flags) {
  FAKE_ENTER("cuMulticastGetGranularity");
  *g = (size_t)4 << 20;
  return CUDA_SUCCESS;
}
CUresult fk_MemCreate(CUmemGenericAllocationHandle* h, size_t, const CUmemAllocationProp*, unsigned long long) {
  FAKE_ENTER("cuMemCreate");
  *h = g_fake.next_handle++;
  g_fake.handles[*h] = 1;
  return CUDA_SUCCESS;
}
CUresult fk_MulticastCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp*) {
  FAKE_ENTER("cuMulticastCreate");
  *h = g_fake.next_handle++;
  g_fake.handles[*h] = 1;
  return CUDA_SUCCESS;
}
CUresult fk_MemRelease(CUmemGenericAllocationHandle h) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  auto it = g_fake.handles.find(h);
  if (it == g_fake.handles.end()) return CUDA_ERROR_INVALID_VALUE;
  if (--it->second == 0) g_fake.handles.erase(it);
  return CUDA_SUCCESS;
}
// The descriptor is a memory file that holds the handle's number.
CUresult fk_MemExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType,
                                       unsigned long long) {
  FAKE_ENTER("cuMemExportToShareableHandle");
  const int fd = memfd_create("bagua-fake-handle", 0);
  if (fd < 0 || pwrite(fd, &h, sizeof(h), 0) != (ssize_t)sizeof(h)) return CUDA_ERROR_UNKNOWN;
  *(int*)out = fd;
  return CUDA_SUCCESS;
}
CUresult fk_MemImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType) {
  FAKE_ENTER("cuMemImportFromShareableHandle");
  const int fd = (int)(uintptr_t)os_handle;
  if (pread(fd, h, sizeof(*h), 0) != (ssize_t)sizeof(*h) || !g_fake.handles.count(*h)) return CUDA_ERROR_INVALID_VALUE;
  g_fake.handles[*h]++;
  return CUDA_SUCCESS;
}
CUresult fk_MemAddressReserve(CUdeviceptr* p, size_t bytes, size_t, CUdeviceptr, unsigned long long) {
  FAKE_ENTER("cuMemAddressReserve");
  *p = g_fake.next_va;
  g_fake.next_va += bytes + ((size_t)64 << 20);
  g_fake.reserved[*p] = bytes;
  return CUDA_SUCCESS;
}
CUresult fk_MemAddressFree(CUdeviceptr p, size_t) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  return g_fake.reserved.erase(p) ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
CUresult fk_MemMap(CUdeviceptr p, size_t, size_t, CUmemGenericAllocationHandle h, unsigned long long) {
  FAKE_ENTER("cuMemMap");
  if (!g_fake.reserved.count(p) || !g_fake.handles.count(h)) return CUDA_ERROR_INVALID_VALUE;
  g_fake.mapped[p] = 1;
  return CUDA_SUCCESS;
}
CUresult fk_MemUnmap(CUdeviceptr p, size_t) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  return g_fake.mapped.erase(p) ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
CUresult fk_MemSetAccess(CUdeviceptr p, size_t, const CUmemAccessDesc*, size_t) {
  FAKE_ENTER("cuMemSetAccess");
  return g_fake.mapped.count(p) ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
CUresult fk_MulticastAddDevice(CUmemGenericAllocationHandle h, CUdevice) {
  FAKE_ENTER("cuMulticastAddDevice");
  return g_fake.handles.count(h) ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
CUresult fk_MulticastBindMem(CUmemGenericAllocationHandle mc, size_t, CUmemGenericAllocationHandle mem, size_t, size_t,
                             unsigned long long) {
  FAKE_ENTER("cuMulticastBindMem");
  if (!g_fake.handles.count(mc) || !g_fake.handles.count(mem)) return CUDA_ERROR_INVALID_VALUE;
  g_fake.bound++;
  return CUDA_SUCCESS;
}
CUresult fk_MulticastUnbind(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  g_fake.bound--;
  return CUDA_SUCCESS;
}

const struct {
  const char* name;
  void* fn;
} kEntries[] = {
    {"cuDeviceGet", (void*)fk_DeviceGet},
    {"cuDeviceGetAttribute", (void*)fk_DeviceGetAttribute},
    {"cuGetErrorString", (void*)fk_GetErrorString},
    {"cuMemGetAllocationGranularity", (void*)fk_MemGetAllocationGranularity},
    {"cuMemCreate", (void*)fk_MemCreate},
    {"cuMemRelease", (void*)fk_MemRelease},
    {"cuMemExportToShareableHandle", (void*)fk_MemExportToShareableHandle},
    {"cuMemImportFromShareableHandle", (void*)fk_MemImportFromShareableHandle},
    {"cuMemAddressReserve", (void*)fk_MemAddressReserve},
    {"cuMemAddressFree", (void*)fk_MemAddressFree},
    {"cuMemMap", (void*)fk_MemMap},
    {"cuMemUnmap", (void*)fk_MemUnmap},
    {"cuMemSetAccess", (void*)fk_MemSetAccess},
    {"cuMulticastCreate", (void*)fk_MulticastCreate},
    {"cuMulticastAddDevice", (void*)fk_MulticastAddDevice},
    {"cuMulticastBindMem", (void*)fk_MulticastBindMem},
    {"cuMulticastUnbind", (void*)fk_MulticastUnbind},
    {"cuMulticastGetGranularity", (void*)fk_MulticastGetGranularity},
};

// ---- stand-in runtime --------------------------------------------------------------------
bool pf_select_device(int) { return true; }
void* pf_driver_entry(const char* name) {
  {
    std::lock_guard<std::mutex> guard(g_fake.mu);
    if (g_fake.fail_rank == t_rank && g_fake.fail_call == std::string("entry:") + name) return nullptr;
  }
  for (const auto& e : kEntries)
    if (std::strcmp(e.name, name) == 0) return e.fn;
  return nullptr;
}
void* pf_alloc(size_t bytes) { return std::malloc(bytes); }
void pf_free(void* p) { std::free(p); }
bool pf_copy(void* dst, const void* src, size_t bytes, cudaStream_t) {
  std::memcpy(dst, src, bytes);
  return true;
}
bool pf_clear(void*, size_t, cudaStream_t) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  return !(g_fake.fail_rank == t_rank && g_fake.fail_call == "clear");
}
const MulticastPlatform kFakePlatform = {pf_select_device, pf_driver_entry, pf_alloc, pf_free, pf_copy, pf_copy, pf_clear};

int open_descriptors() {
  int n = 0;
  if (DIR* d = opendir("/proc/self/fd")) {
    while (readdir(d)) ++n;
    closedir(d);
  }
  return n;
}

struct Outcome {
  bool ok = false;
  std::string why;
  MulticastSlab slab;
};

// One collective set-up on `nranks` threads; the slabs are destroyed unless `keep` is given.
std::vector<Outcome> run_setup(int nranks, size_t bytes, std::vector<MulticastSlab>* keep = nullptr) {
  Hub hub(nranks);
  std::vector<Outcome> out((size_t)nranks);
  std::vector<std::thread> threads;
  for (int r = 0; r < nranks; ++r)
    threads.emplace_back([&, r] {
      t_rank = r;
      ThreadTransport transport(hub, r);
      Outcome& o = out[(size_t)r];
      o.ok = create_multicast_slab(transport, r, nranks, r, nullptr, bytes, &o.slab, &o.why);
    });
  for (auto& t : threads) t.join();
  if (keep) {
    for (auto& o : out) keep->push_back(o.slab);
  } else {
    for (auto& o : out) destroy_multicast_slab(o.slab);
  }
  return out;
}

int g_failures = 0;
void expect(bool cond, const std::string& what) {
  if (!cond) {
    std::fprintf(stderr, "FAILED: %s\n", what.c_str());
    ++g_failures;
  }
}
void expect_nothing_left(const std::string& where) {
  std::lock_guard<std::mutex> guard(g_fake.mu);
  expect(g_fake.handles.empty(), where + ": " + std::to_string(g_fake.handles.size()) + " handles still referenced");
  expect(g_fake.reserved.empty(), where + ": address ranges still reserved");
  expect(g_fake.mapped.empty(), where + ": mappings left");
  expect(g_fake.bound == 0, where + ": bindings left (" + std::to_string(g_fake.bound) + ")");
}

}  // namespace

int main(int argc, char** argv) {
  const bool verbose = argc > 1 && std::string(argv[1]) == "-v";
  set_multicast_platform(&kFakePlatform);
  const int fds_at_start = open_descriptors();
  int cases = 0;

  // 1. healthy stand-in
  for (int n : {2, 4, 8}) {
    std::vector<MulticastSlab> slabs;
    const auto out = run_setup(n, ((size_t)5 << 20) + 3, &slabs);
    for (int r = 0; r < n; ++r) {
      const Outcome& o = out[(size_t)r];
      expect(o.ok, "healthy set-up on " + std::to_string(n) + " ranks, rank " + std::to_string(r) + ": " + o.why);
      expect(o.slab.bytes == ((size_t)8 << 20), "size rounded up to the larger granularity");
      expect(o.slab.mc_base != nullptr, "multicast mapping present");
      for (int p = 0; p < n; ++p) {
        expect(o.slab.base[p] != nullptr, "mapping of every rank's memory");
        for (int q = 0; q < p; ++q) expect(o.slab.base[p] != o.slab.base[q], "mappings are distinct");
      }
    }
    {
      std::lock_guard<std::mutex> guard(g_fake.mu);
      expect((int)g_fake.handles.size() == n + 1, "one allocation per rank and one multicast object");
      for (auto& kv : g_fake.handles) expect(kv.second == n, "every handle is held once by every rank");
      expect((int)g_fake.mapped.size() == n * (n + 1) && g_fake.bound == n, "mappings and bindings of a live slab");
    }
    expect(open_descriptors() == fds_at_start, "descriptors are closed once every peer has imported them");
    for (auto& s : slabs) destroy_multicast_slab(s);
    expect_nothing_left("after destroying a healthy slab");
    ++cases;
  }

  // 2. every driver call failing on the first or on the last rank
  const char* calls[] = {"cuDeviceGet", "cuDeviceGetAttribute", "cuMulticastGetGranularity", "cuMemGetAllocationGranularity",
                         "cuMulticastCreate", "cuMemCreate", "cuMemExportToShareableHandle",
                         "cuMemImportFromShareableHandle", "cuMulticastAddDevice", "cuMulticastBindMem",
                         "cuMemAddressReserve", "cuMemMap", "cuMemSetAccess", "clear", "entry:cuMulticastBindMem"};
  for (const char* call : calls)
    for (int n : {2, 5})
      for (int bad_rank : {0, n - 1}) {
        if (std::string(call) == "cuMulticastCreate" && bad_rank != 0) continue;  // only rank 0 creates the object
        {
          std::lock_guard<std::mutex> guard(g_fake.mu);
          g_fake.fail_call = call;
          g_fake.fail_rank = bad_rank;
        }
        const auto out = run_setup(n, (size_t)1 << 20);
        const std::string label = std::string(call) + " failing on rank " + std::to_string(bad_rank) + " of " + std::to_string(n);
        const std::string marker = " failed on rank " + std::to_string(bad_rank);
        const std::string step = out[0].why.substr(0, out[0].why.find(marker));
        for (int r = 0; r < n; ++r) {
          expect(!out[(size_t)r].ok, label + ": rank " + std::to_string(r) + " must not get a slab");
          expect(out[(size_t)r].why.find(marker) != std::string::npos,
                 label + ": rank " + std::to_string(r) + " blames the right rank (" + out[(size_t)r].why + ")");
          expect(out[(size_t)r].why.substr(0, step.size()) == step, label + ": all ranks stop at the same step");
          expect(out[(size_t)r].slab.impl == nullptr && out[(size_t)r].slab.mc_base == nullptr, label + ": no slab handed out");
        }
        expect_nothing_left(label);
        expect(open_descriptors() == fds_at_start, label + ": descriptors leaked");
        if (verbose) std::printf("%s -> rank 0: %s | rank %d: %s\n", label.c_str(), out[0].why.c_str(), n - 1, out[(size_t)n - 1].why.c_str());
        ++cases;
      }
  {
    std::lock_guard<std::mutex> guard(g_fake.mu);
    g_fake.fail_call.clear();
    g_fake.fail_rank = -1;
    g_fake.multicast_supported = false;
  }
  {
    const auto out = run_setup(3, (size_t)1 << 20);
    for (auto& o : out) expect(!o.ok && o.why.find("capability check") == 0, "a device without multicast support: " + o.why);
    expect_nothing_left("no multicast support");
    std::lock_guard<std::mutex> guard(g_fake.mu);
    g_fake.multicast_supported = true;
    ++cases;
  }

  // 3. dropping the bindings at process exit, then the ordinary destruction
  {
    std::vector<MulticastSlab> slabs;
    const auto out = run_setup(4, (size_t)1 << 20, &slabs);
    for (auto& o : out) expect(o.ok, "set-up before release_all: " + o.why);
    expect(release_all_multicast_slabs() == 4, "release_all_multicast_slabs() reports the live slabs");
    expect_nothing_left("after release_all_multicast_slabs");
    expect(release_all_multicast_slabs() == 0, "a second call finds nothing");
    for (auto& s : slabs) destroy_multicast_slab(s);
    expect_nothing_left("destroy after release_all");
    ++cases;
  }
  expect(open_descriptors() == fds_at_start, "descriptors at the end");

  set_multicast_platform(nullptr);
  std::printf("multicast slab set-up: %d cases, %d driver calls, %d failures\n", cases, g_fake.calls, g_failures);
  return g_failures ? 1 : 0;
}
