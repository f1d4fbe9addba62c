#include "arena.h"

#include <cuda_runtime.h>

namespace bagua {

namespace {
struct HandlePair {
  cudaIpcMemHandle_t staging;
  cudaIpcMemHandle_t signals;
  uint64_t staging_bytes;
  uint64_t has_signals;  // signals handle is only exchanged once
};
static_assert(sizeof(HandlePair) == 144, "unexpected IPC handle size");
}  // namespace

PeerArena::PeerArena(Transport& transport, int rank, int nranks, int device, cudaStream_t stream)
    : transport_(transport), rank_(rank), nranks_(nranks), device_(device), stream_(stream) {
  BAGUA_CHECK(nranks <= kArenaMaxRanks, Communicator,
              "the peer arena supports at most " << kArenaMaxRanks << " ranks, got " << nranks);
  deadline_ns_ = (uint64_t)(env_double("BAGUA_B200_DEVICE_WAIT_MS", 120000.0) * 1e6);
  max_blocks_ = (int)std::min<long>(std::max<long>(env_long("BAGUA_B200_COMM_CTAS", 64), 1), kArenaMaxBlocks);
  max_coop_blocks_ = (int)std::min<long>(std::max<long>(env_long("BAGUA_B200_COOP_CTAS", 148), 1), kArenaMaxBlocks);
  nvls_ = env_long("BAGUA_B200_NVLS", 0) != 0;
  BAGUA_CUDA_CHECK(cudaSetDevice(device));
  try {
    BAGUA_CUDA_CHECK(cudaMalloc(&local_signals_, kSigWords * sizeof(uint32_t)));
    BAGUA_CUDA_CHECK(cudaMemset(local_signals_, 0, kSigWords * sizeof(uint32_t)));
    static_assert(sizeof(DeviceStatus) <= 60, "the status record shares 64 bytes with the poison source word");
    BAGUA_CUDA_CHECK(cudaHostAlloc((void**)&status_host_, 64, cudaHostAllocMapped));
    std::memset(status_host_, 0, 64);
    reinterpret_cast<uint32_t*>(status_host_)[15] = 1u;  // what poison() copies into the pad
    BAGUA_CUDA_CHECK(cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0));
    BAGUA_CUDA_CHECK(cudaStreamCreateWithFlags(&abort_stream_, cudaStreamNonBlocking));
    BAGUA_CUDA_CHECK(cudaDeviceSynchronize());
    // fails when a peer cannot be mapped (no peer access between the devices, IPC disabled)
    allocate_and_exchange((size_t)env_long("BAGUA_B200_STAGING_MB", 64) << 20);
  } catch (...) {
    release();  // a constructor that throws gets no destructor call
    throw;
  }
}

PeerArena::~PeerArena() { release(); }

void PeerArena::release() {
  // Best effort; at interpreter shutdown the runtime may already be gone.
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    if (peer_staging_[p]) cudaIpcCloseMemHandle(peer_staging_[p]);
    if (peer_signals_[p]) cudaIpcCloseMemHandle(peer_signals_[p]);
  }
  for (void* p : retired_peer_) cudaIpcCloseMemHandle(p);
  for (Slab& s : slabs_) {
    if (s.vmm.impl) {
      destroy_multicast_slab(s.vmm);
      continue;
    }
    for (int p = 0; p < nranks_; ++p) {
      if (!s.base[p]) continue;
      if (p == rank_)
        cudaFree(s.base[p]);
      else
        cudaIpcCloseMemHandle(s.base[p]);
    }
  }
  slabs_.clear();
  retired_peer_.clear();
  if (local_staging_) cudaFree(local_staging_);
  for (void* p : retired_) cudaFree(p);
  retired_.clear();
  if (abort_stream_) {
    cudaStreamSynchronize(abort_stream_);  // a poison() copy still reads status_host_
    cudaStreamDestroy(abort_stream_);
    abort_stream_ = nullptr;
  }
  if (local_signals_) cudaFree(local_signals_);
  if (status_host_) cudaFreeHost(status_host_);
  local_staging_ = nullptr;
  local_signals_ = nullptr;
  status_host_ = nullptr;
  for (int p = 0; p < kArenaMaxRanks; ++p) peer_staging_[p] = peer_signals_[p] = nullptr;
  cudaGetLastError();
}

void PeerArena::allocate_and_exchange(size_t bytes) {
  bytes = align_up(bytes, (size_t)2 << 20);
  const bool first = (local_staging_ == nullptr);
  // Everything queued on the stream so far may still use the old staging.
  BAGUA_CUDA_CHECK(cudaStreamSynchronize(stream_));
  void* fresh = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc(&fresh, bytes));
  // until `fresh` becomes the arena's staging, an exception must give it back
  struct FreeOnError {
    void*& p;
    ~FreeOnError() {
      if (p) cudaFree(p);
    }
  } guard{fresh};

  HandlePair mine;
  std::memset(&mine, 0, sizeof(mine));
  BAGUA_CUDA_CHECK(cudaIpcGetMemHandle(&mine.staging, fresh));
  mine.staging_bytes = bytes;
  if (first) {
    BAGUA_CUDA_CHECK(cudaIpcGetMemHandle(&mine.signals, local_signals_));
    mine.has_signals = 1;
  }
  // all-gather the handles through the library transport (device buffers)
  void* dev = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc(&dev, sizeof(HandlePair) * (size_t)nranks_));
  BAGUA_CUDA_CHECK(cudaMemcpyAsync((char*)dev + sizeof(HandlePair) * (size_t)rank_, &mine, sizeof(mine),
                                   cudaMemcpyHostToDevice, stream_));
  transport_.allgather((char*)dev + sizeof(HandlePair) * (size_t)rank_, dev, (int64_t)sizeof(HandlePair), DType::U8);
  std::vector<HandlePair> all((size_t)nranks_);
  BAGUA_CUDA_CHECK(cudaMemcpyAsync(all.data(), dev, sizeof(HandlePair) * (size_t)nranks_, cudaMemcpyDeviceToHost,
                                   stream_));
  BAGUA_CUDA_CHECK(cudaStreamSynchronize(stream_));
  BAGUA_CUDA_CHECK(cudaFree(dev));

  for (int p = 0; p < nranks_; ++p) {
    BAGUA_CHECK(all[p].staging_bytes == bytes, Communicator,
                "ranks disagree on the staging size (" << all[p].staging_bytes << " vs " << bytes
                                                       << "); fused ops must be issued identically on every rank");
    if (p == rank_) continue;
    if (peer_staging_[p]) retired_peer_.push_back(peer_staging_[p]);
    void* mapped = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[p].staging, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      throw BaguaError(ErrorKind::Communicator, std::string("cannot map the staging buffer of rank ") +
                                                    std::to_string(p) + ": " + cudaGetErrorString(e));
    }
    peer_staging_[p] = mapped;
    if (first) {
      e = cudaIpcOpenMemHandle(&mapped, all[p].signals, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        cudaGetLastError();
        throw BaguaError(ErrorKind::Communicator, std::string("cannot map the signal pad of rank ") +
                                                      std::to_string(p) + ": " + cudaGetErrorString(e));
      }
      peer_signals_[p] = mapped;
    }
  }
  if (local_staging_) retired_.push_back(local_staging_);
  local_staging_ = fresh;
  peer_staging_[rank_] = fresh;
  fresh = nullptr;  // owned by the arena from here on
  peer_signals_[rank_] = local_signals_;
  staging_bytes_ = bytes;
  // Nobody may write into the new staging before every rank has mapped it.
  transport_.barrier();
  BAGUA_LOG(Info, "peer arena rank " << rank_ << "/" << nranks_ << ": staging " << (bytes >> 20) << " MiB mapped");
}

void PeerArena::exchange_block(size_t bytes, void** local, void* peers[kArenaMaxRanks]) {
  BAGUA_CUDA_CHECK(cudaSetDevice(device_));
  void* fresh = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc(&fresh, bytes));
  BAGUA_CUDA_CHECK(cudaMemset(fresh, 0, bytes));
  struct Msg {
    cudaIpcMemHandle_t handle;
    uint64_t bytes;
  } mine;
  std::memset(&mine, 0, sizeof(mine));
  BAGUA_CUDA_CHECK(cudaIpcGetMemHandle(&mine.handle, fresh));
  mine.bytes = bytes;
  void* dev = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc(&dev, sizeof(Msg) * (size_t)nranks_));
  BAGUA_CUDA_CHECK(cudaMemcpyAsync((char*)dev + sizeof(Msg) * (size_t)rank_, &mine, sizeof(mine),
                                   cudaMemcpyHostToDevice, stream_));
  transport_.allgather((char*)dev + sizeof(Msg) * (size_t)rank_, dev, (int64_t)sizeof(Msg), DType::U8);
  std::vector<Msg> all((size_t)nranks_);
  BAGUA_CUDA_CHECK(cudaMemcpyAsync(all.data(), dev, sizeof(Msg) * (size_t)nranks_, cudaMemcpyDeviceToHost, stream_));
  BAGUA_CUDA_CHECK(cudaStreamSynchronize(stream_));
  BAGUA_CUDA_CHECK(cudaFree(dev));
  for (int p = 0; p < nranks_; ++p) {
    BAGUA_CHECK(all[p].bytes == bytes, Communicator,
                "ranks disagree on a symmetric allocation (" << all[p].bytes << " vs " << bytes
                                                             << " bytes); allocate identically on every rank");
    if (p == rank_) {
      peers[p] = fresh;
      continue;
    }
    void* mapped = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[p].handle, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      throw BaguaError(ErrorKind::Communicator, std::string("cannot map symmetric memory of rank ") +
                                                    std::to_string(p) + ": " + cudaGetErrorString(e));
    }
    peers[p] = mapped;
  }
  *local = fresh;
  transport_.barrier();
}

void* PeerArena::sym_alloc(size_t bytes) {
  std::lock_guard<std::mutex> g(sym_mu_);
  bytes = align_up(bytes == 0 ? 1 : bytes, 256);
  if (slabs_.empty() || slabs_.back().used + bytes > slabs_.back().bytes) {
    static const size_t slab_min = (size_t)env_long("BAGUA_B200_SYM_SLAB_MB", 256) << 20;
    const size_t slab_bytes = align_up(std::max(bytes, slab_min), (size_t)2 << 20);
    Slab s{};
    bool made = false;
    if (nvls_) {
      // Collective, and all ranks get the same answer: a slab with a multicast mapping or none.
      std::string why;
      BAGUA_CUDA_CHECK(cudaSetDevice(device_));
      made = create_multicast_slab(transport_, rank_, nranks_, device_, stream_, slab_bytes, &s.vmm, &why);
      if (made) {
        for (int p = 0; p < nranks_; ++p) s.base[p] = s.vmm.base[p];
        s.mc_base = s.vmm.mc_base;
        s.bytes = s.vmm.bytes;
        BAGUA_LOG(Info, "symmetric slab of " << (s.bytes >> 20) << " MiB with an NVSwitch multicast mapping");
      } else {
        BAGUA_LOG(Warn, "NVSwitch multicast is not usable, symmetric memory falls back to CUDA IPC: " << why);
        nvls_ = false;
      }
    }
    if (!made) {
      void* local = nullptr;
      void* peers[kArenaMaxRanks] = {};
      exchange_block(slab_bytes, &local, peers);
      for (int p = 0; p < nranks_; ++p) s.base[p] = (char*)peers[p];
      s.bytes = slab_bytes;
    }
    s.used = 0;
    slabs_.push_back(s);
  }
  Slab& s = slabs_.back();
  void* out = s.base[rank_] + s.used;
  s.used += bytes;
  sym_used_ += bytes;
  return out;
}

bool PeerArena::sym_translate(const void* p, size_t bytes, void* peers[kArenaMaxRanks]) const {
  std::lock_guard<std::mutex> g(sym_mu_);
  const char* c = (const char*)p;
  for (const Slab& s : slabs_) {
    const char* b = s.base[rank_];
    if (c >= b && c + bytes <= b + s.used) {
      for (int q = 0; q < nranks_; ++q) peers[q] = s.base[q] + (c - b);
      return true;
    }
  }
  return false;
}

void* PeerArena::sym_multicast(const void* p, size_t bytes) const {
  std::lock_guard<std::mutex> g(sym_mu_);
  const char* c = (const char*)p;
  for (const Slab& s : slabs_) {
    const char* b = s.base[rank_];
    if (s.mc_base && c >= b && c + bytes <= b + s.used) return s.mc_base + (c - b);
  }
  return nullptr;
}

void PeerArena::ensure_staging(size_t bytes) {
  if (bytes <= staging_bytes_) return;
  size_t want = staging_bytes_ ? staging_bytes_ : ((size_t)64 << 20);
  while (want < bytes) want <<= 1;
  allocate_and_exchange(want);
}

ArenaView PeerArena::next_view(int grid, int grid_barriers) {
  ArenaView v;
  std::memset(&v, 0, sizeof(v));
  for (int p = 0; p < nranks_; ++p) {
    v.staging[p] = (uint8_t*)peer_staging_[p];
    v.signals[p] = (uint32_t*)peer_signals_[p];
  }
  v.status = status_dev_;
  v.staging_bytes = staging_bytes_;
  v.rank = rank_;
  v.nranks = nranks_;
  v.epoch = ++epoch_;
  v.deadline_ns = deadline_ns_;
  v.grid_bar_base = grid_bar_;
  grid_bar_ += (uint64_t)grid * (uint64_t)grid_barriers;
  return v;
}

DeviceStatus PeerArena::read_status() const {
  DeviceStatus s;
  std::memcpy(&s, (const void*)status_host_, sizeof(s));
  return s;
}
void PeerArena::clear_status() { std::memset(status_host_, 0, sizeof(DeviceStatus)); }

void PeerArena::poison() {
  if (!local_signals_ || !abort_stream_) return;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  // pinned source, stream of its own: queues behind nothing and does not wait for running kernels
  cudaError_t e = cudaMemcpyAsync((uint32_t*)local_signals_ + kSigPoison, reinterpret_cast<uint32_t*>(status_host_) + 15,
                                  sizeof(uint32_t), cudaMemcpyHostToDevice, abort_stream_);
  if (e != cudaSuccess) {
    cudaGetLastError();
    BAGUA_LOG(Warn, "could not raise the device-side abort word: " << cudaGetErrorString(e));
  }
  cudaSetDevice(prev);
}

}  // namespace bagua
