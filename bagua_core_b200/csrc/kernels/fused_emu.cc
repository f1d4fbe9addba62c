// Host side of the single-GPU emulation of the fused kernels (see fused_emu.h).
#include "fused_emu.h"

#include <cuda_runtime.h>

namespace bagua {
namespace fused {

namespace {
constexpr int kHdr = 32;
size_t elem_bytes(DType dt) { return dtype_bytes(dt); }
}  // namespace

EmulatedArena::EmulatedArena(int nranks, int device, size_t staging_bytes)
    : nranks_(nranks), device_(device), staging_bytes_(align_up(staging_bytes, 256)) {
  BAGUA_CHECK(nranks >= 2 && nranks <= kArenaMaxRanks, Communicator, "emulation supports 2.." << kArenaMaxRanks << " ranks");
  BAGUA_CUDA_CHECK(cudaSetDevice(device));
  for (int r = 0; r < nranks; ++r) {
    void* s = nullptr;
    void* p = nullptr;
    BAGUA_CUDA_CHECK(cudaMalloc(&s, staging_bytes_));
    BAGUA_CUDA_CHECK(cudaMalloc(&p, kSigWords * sizeof(uint32_t)));
    BAGUA_CUDA_CHECK(cudaMemset(p, 0, kSigWords * sizeof(uint32_t)));
    staging_.push_back(s);
    signals_.push_back(p);
  }
  BAGUA_CUDA_CHECK(cudaHostAlloc((void**)&status_host_, sizeof(DeviceStatus), cudaHostAllocMapped));
  std::memset(status_host_, 0, sizeof(DeviceStatus));
  BAGUA_CUDA_CHECK(cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0));
  BAGUA_CUDA_CHECK(cudaMalloc((void**)&dev_args_, sizeof(EmuRank) * (size_t)nranks));
  BAGUA_CUDA_CHECK(cudaDeviceSynchronize());
}

EmulatedArena::~EmulatedArena() {
  for (void* p : staging_) cudaFree(p);
  for (void* p : signals_) cudaFree(p);
  if (dev_args_) cudaFree(dev_args_);
  if (status_host_) cudaFreeHost(status_host_);
  cudaGetLastError();
}

EmuRank* EmulatedArena::prepare(std::vector<EmuRank>& host, int blocks, int grid_barriers, size_t staging_needed) {
  BAGUA_CHECK(blocks >= 1 && blocks <= kArenaMaxBlocks, Communicator, "emulation: blocks per rank out of range");
  BAGUA_CHECK(staging_needed <= staging_bytes_, Communicator,
              "emulation: op needs " << staging_needed << " bytes of staging per rank, arena has " << staging_bytes_);
  BAGUA_CHECK((int)host.size() == nranks_, Communicator, "emulation: one entry per rank expected");
  BAGUA_CUDA_CHECK(cudaSetDevice(device_));
  ++epoch_;
  for (int r = 0; r < nranks_; ++r) {
    ArenaView& v = host[r].view;
    std::memset(&v, 0, sizeof(v));
    for (int q = 0; q < nranks_; ++q) {
      v.staging[q] = (uint8_t*)staging_[q];
      v.signals[q] = (uint32_t*)signals_[q];
    }
    v.status = status_dev_;
    v.staging_bytes = staging_bytes_;
    v.rank = r;
    v.nranks = nranks_;
    v.epoch = epoch_;
    v.deadline_ns = deadline_ns_;
    v.grid_bar_base = grid_bar_;
  }
  grid_bar_ += (uint64_t)blocks * (uint64_t)grid_barriers;  // every virtual rank's counter advances alike
  BAGUA_CUDA_CHECK(cudaMemcpy(dev_args_, host.data(), sizeof(EmuRank) * (size_t)nranks_, cudaMemcpyHostToDevice));
  return dev_args_;
}

void EmulatedArena::finish(const char* what) {
  BAGUA_CUDA_CHECK(cudaGetLastError());
  BAGUA_CUDA_CHECK(cudaDeviceSynchronize());
  DeviceStatus s;
  std::memcpy(&s, (const void*)status_host_, sizeof(s));
  if (s.code != 0) {
    std::ostringstream o;
    o << "emulated " << what << ": a device-side wait ran out (code " << s.code << ", phase " << s.phase << ", peer "
      << s.peer << ", block " << s.block << ", epoch " << s.epoch << ", last value seen " << s.seen << ")";
    throw BaguaError(ErrorKind::Communicator, o.str());
  }
}

void EmulatedArena::allreduce(const std::vector<const void*>& in, const std::vector<void*>& out, int64_t n, DType dt,
                              float scale, EmuAllreduceMode mode, int blocks) {
  const size_t bytes = (size_t)n * elem_bytes(dt);
  BAGUA_CHECK(bytes % 16 == 0 && (int)in.size() == nranks_ && (int)out.size() == nranks_, Tensor,
              "emulated all-reduce: need one 16-byte-multiple buffer per rank");
  const int64_t nvec = (int64_t)(bytes / 16);
  std::vector<EmuRank> host((size_t)nranks_);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  size_t need = 0;
  int64_t aux = 0;
  if (mode == EmuAllreduceMode::OneShot) {
    need = (size_t)nranks_ * bytes;
    aux = nvec;
  } else if (mode == EmuAllreduceMode::TwoShot) {
    aux = (nvec + nranks_ - 1) / nranks_;
    need = ((size_t)nranks_ * (size_t)aux + (size_t)nvec) * 16;
  }
  for (int r = 0; r < nranks_; ++r) {
    BAGUA_CHECK((uintptr_t)in[r] % 16 == 0 && (uintptr_t)out[r] % 16 == 0, Tensor, "buffers must be 16-byte aligned");
    host[r].in = in[r];
    host[r].out = out[r];
    for (int q = 0; q < nranks_; ++q) {
      host[r].sym_in[q] = in[q];
      host[r].sym_out[q] = out[q];
    }
  }
  EmuRank* dev = prepare(host, blocks, 0, need);
  if (mode == EmuAllreduceMode::SymmetricTma)
    emu_launch_allreduce_tma(dev, nranks_, blocks, n, dt, scale);
  else
    emu_launch_allreduce(dev, nranks_, blocks, n, dt, scale, mode, aux);
  finish("all-reduce");
}

void EmulatedArena::pair_average(const std::vector<const void*>& in, const std::vector<void*>& out, int64_t n, DType dt,
                                 const std::vector<int>& peers, int blocks, bool symmetric) {
  const size_t bytes = (size_t)n * elem_bytes(dt);
  BAGUA_CHECK(bytes % 16 == 0 && (int)in.size() == nranks_ && (int)out.size() == nranks_ && (int)peers.size() == nranks_,
              Tensor, "emulated pair average: need one buffer and one peer per rank");
  std::vector<EmuRank> host((size_t)nranks_);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  for (int r = 0; r < nranks_; ++r) {
    BAGUA_CHECK(peers[r] >= 0 && peers[r] < nranks_ && peers[r] != r && peers[peers[r]] == r, Communicator,
                "pairs must be mutual");
    host[r].in = in[r];
    host[r].out = out[r];
    host[r].peer = peers[r];
    for (int q = 0; q < nranks_; ++q) host[r].sym_in[q] = in[q];
  }
  EmuRank* dev = prepare(host, blocks, 0, symmetric ? 0 : bytes);
  emu_launch_pair_average(dev, nranks_, blocks, n, dt, symmetric);
  finish("pair average");
}

void EmulatedArena::collective(EmuCollective kind, const std::vector<const void*>& in, const std::vector<void*>& out,
                               size_t chunk_bytes, DType dt, float scale, int root, bool symmetric, int blocks) {
  std::vector<EmuRank> host((size_t)nranks_);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  const size_t N = (size_t)nranks_;
  size_t need = 0;
  int aux = 0;
  if (kind == EmuCollective::Barrier) {
    blocks = 1;
  } else {
    BAGUA_CHECK(chunk_bytes > 0 && chunk_bytes % 16 == 0 && out.size() == N, Tensor,
                "emulated collective: need one 16-byte-multiple buffer per rank");
    const bool bcast = kind == EmuCollective::BroadcastDirect || kind == EmuCollective::BroadcastTwoPhase;
    const bool rooted = kind == EmuCollective::Scatter || kind == EmuCollective::Gather ||
                        kind == EmuCollective::ReduceDirect || kind == EmuCollective::ReduceTwoPhase;
    if (bcast) {
      BAGUA_CHECK(root >= 0 && root < nranks_, Communicator, "emulated broadcast: root out of range");
      need = chunk_bytes;
      aux = root;
    } else if (rooted) {
      BAGUA_CHECK(root >= 0 && root < nranks_ && in.size() == N, Communicator,
                  "emulated rooted collective: root out of range or inputs missing");
      const size_t nvec = chunk_bytes / 16;
      bool in_place = false;
      if (kind == EmuCollective::Scatter) {
        need = chunk_bytes;
        in_place = (const char*)out[(size_t)root] == (const char*)in[(size_t)root] + (size_t)root * chunk_bytes;
      } else if (kind == EmuCollective::Gather) {
        need = N * chunk_bytes;
        in_place = (const char*)in[(size_t)root] == (const char*)out[(size_t)root] + (size_t)root * chunk_bytes;
      } else if (kind == EmuCollective::ReduceDirect) {
        need = N * chunk_bytes;
      } else {
        need = (N * ((nvec + N - 1) / N) + nvec) * 16;
      }
      aux = root | (in_place ? 1 << 8 : 0);
    } else {
      BAGUA_CHECK(in.size() == N, Tensor, "emulated collective: one input per rank expected");
      need = symmetric ? 0 : N * chunk_bytes;
      bool in_place = true;
      for (size_t r = 0; r < N; ++r) {
        const char* local = kind == EmuCollective::AllToAll ? (const char*)out[r] : (const char*)out[r] + r * chunk_bytes;
        in_place = in_place && (const char*)in[r] == local;
      }
      if (kind == EmuCollective::ReduceScatter) in_place = false;
      BAGUA_CHECK(!(symmetric && kind == EmuCollective::AllToAll && in_place), Tensor,
                  "an in-place all-to-all cannot store into the peers' buffers directly");
      aux = (symmetric ? 1 : 0) | (in_place ? 2 : 0);
    }
    for (size_t r = 0; r < N; ++r) {
      BAGUA_CHECK((uintptr_t)out[r] % 16 == 0 && (bcast || (uintptr_t)in[r] % 16 == 0), Tensor,
                  "buffers must be 16-byte aligned");
      host[r].in = bcast ? nullptr : in[r];
      host[r].out = out[r];
      for (size_t q = 0; q < N; ++q) {
        host[r].sym_in[q] = bcast ? nullptr : in[q];
        host[r].sym_out[q] = out[q];
      }
    }
  }
  EmuRank* dev = prepare(host, blocks, 0, need);
  emu_launch_collective(dev, nranks_, blocks, kind, (int64_t)(chunk_bytes / 16), dt, aux, scale);
  finish("collective");
}

void EmulatedArena::alltoall_v(const std::vector<const void*>& in, const std::vector<void*>& out,
                               const std::vector<int64_t>& bytes, int blocks) {
  const size_t N = (size_t)nranks_;
  BAGUA_CHECK(in.size() == N && out.size() == N && bytes.size() == N * N, Tensor,
              "emulated alltoall_v: one input and output per rank and an N x N size table expected");
  // the layout of fused::collectives::VSegments: four arrays of kArenaMaxRanks 64-bit words
  struct Segments {
    int64_t send_off[kArenaMaxRanks], send_bytes[kArenaMaxRanks], recv_off[kArenaMaxRanks], recv_bytes[kArenaMaxRanks];
  };
  std::vector<Segments> seg(N);
  std::vector<EmuRank> host(N);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  for (size_t r = 0; r < N; ++r) {
    std::memset(&seg[r], 0, sizeof(Segments));
    int64_t so = 0, ro = 0;
    for (size_t q = 0; q < N; ++q) {
      BAGUA_CHECK(bytes[r * N + q] >= 0, Tensor, "emulated alltoall_v: negative size");
      seg[r].send_off[q] = so;
      seg[r].send_bytes[q] = bytes[r * N + q];
      so += bytes[r * N + q];
      seg[r].recv_off[q] = ro;
      seg[r].recv_bytes[q] = bytes[q * N + r];
      ro += bytes[q * N + r];
    }
    host[r].in = in[r];
    host[r].out = out[r];
    for (size_t q = 0; q < N; ++q) host[r].sym_in[q] = in[q];
  }
  EmuRank* dev = prepare(host, blocks, 0, N * 16);
  void* dseg = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc(&dseg, sizeof(Segments) * N));
  cudaError_t e = cudaMemcpy(dseg, seg.data(), sizeof(Segments) * N, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    try {
      emu_launch_alltoall_v(dev, dseg, nranks_, blocks);
      finish("alltoall_v");
    } catch (...) {
      cudaFree(dseg);
      throw;
    }
  }
  cudaFree(dseg);
  BAGUA_CUDA_CHECK(e);
}

void EmulatedArena::bytegrad(const std::vector<void*>& buckets, int64_t n, DType dt, bool average, int blocks) {
  BAGUA_CHECK((int)buckets.size() == nranks_ && n % ((int64_t)16 * nranks_) == 0, Tensor,
              "emulated ByteGrad: n must be a multiple of 16 * nranks");
  const int64_t chunk = n / nranks_;
  const size_t slot = (size_t)chunk + kHdr;
  const size_t scratch_off = align_up(2 * (size_t)nranks_ * slot, 256);
  std::vector<EmuRank> host((size_t)nranks_);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  for (int r = 0; r < nranks_; ++r) host[r].in = buckets[r];
  EmuRank* dev = prepare(host, blocks, 2, scratch_off + (size_t)(nranks_ + 1) * blocks * sizeof(float2));
  emu_launch_bytegrad(dev, nranks_, blocks, n, dt, average ? 1.0f / (float)nranks_ : 1.0f, slot, scratch_off);
  finish("ByteGrad");
}

void EmulatedArena::lp_ring(const std::vector<void*>& x, const std::vector<void*>& w, const std::vector<void*>& l,
                            const std::vector<void*>& r, int64_t n, DType dt, int blocks) {
  BAGUA_CHECK((int)x.size() == nranks_ && (int)w.size() == nranks_ && (int)l.size() == nranks_ &&
                  (int)r.size() == nranks_ && n % 16 == 0,
              Tensor, "emulated low-precision ring: n must be a multiple of 16, one buffer per rank");
  const size_t slot = (size_t)n + kHdr;
  const size_t scratch_off = align_up(3 * slot, 256);
  std::vector<EmuRank> host((size_t)nranks_);
  for (auto& h : host) std::memset(&h, 0, sizeof(h));
  for (int k = 0; k < nranks_; ++k) {
    host[k].in = x[k];
    host[k].w = w[k];
    host[k].l = l[k];
    host[k].r = r[k];
  }
  EmuRank* dev = prepare(host, blocks, 1, scratch_off + (size_t)blocks * sizeof(float2));
  emu_launch_lp_ring(dev, nranks_, blocks, n, dt, slot, scratch_off);
  finish("low-precision ring");
}

}  // namespace fused
}  // namespace bagua
