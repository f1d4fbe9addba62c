// Fused all-reduce (+scale) and pair-average over peer memory, sm_100a.
//
// One launch per bucket, no library collective.  Work is cut in 16-byte vectors; block b
// of every rank owns the same vector range, so blocks pair up across GPUs through
// per-block signal words and never need a grid-wide barrier.
//
//   one-shot  (small buffers): every rank stores its slice into slot[rank] of every
//             peer's staging, signals, waits for the N-1 signals addressed to it, and sums
//             the N contributions in rank order (bit-identical on all ranks).
//             Wire per GPU: (N-1)·S out.  One signalling hop.
//   two-shot  (large buffers): reduce-scatter by push (chunk q of my data → slot[me] of
//             q's staging), owner sums chunk `me` in rank order, scales, and stores the
//             result both locally and into every peer's all-gather area; peers copy it
//             out of their own staging.  Wire per GPU: 2(N-1)/N·S out.  Two hops.
//   symmetric (large buffers in the symmetric heap): no staging; rank r loads chunk r of
//             all N inputs directly, reduces, and stores into chunk r of all N outputs.
//
// Accumulation is fp32 for every dtype, rounded once.  Each algorithm is a `*_body`
// device function; the `__global__` kernels only supply the block's position (`Launch`),
// which lets the single-GPU emulation run exactly the same code for all ranks at once.
#include <cuda_runtime.h>

#include "fused.h"
#include "fused_emu.h"
#include "fused_allreduce_bodies.cuh"
#include "fused_allreduce_tma.cuh"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {

namespace {

using psync::Launch;
using namespace allreduce_bodies;


// ---- real kernels: one launch per rank ---------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    pair_average_sym_kernel(const __grid_constant__ ArenaView v, const uint4* __restrict__ in,
                            const uint4* __restrict__ peer_in, uint4* __restrict__ out, int64_t nvec, int peer) {
  pair_average_sym_body<T>(v, psync::real_launch(), in, peer_in, out, nvec, peer);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    allreduce_oneshot_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t nvec,
                             int64_t slot_vecs, float scale) {  // in == out for the in-place call
  allreduce_oneshot_body<T>(v, psync::real_launch(), in, out, nvec, slot_vecs, scale);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    allreduce_twoshot_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t nvec,
                             int64_t max_chunk_vecs, float scale) {  // in == out for the in-place call
  allreduce_twoshot_body<T>(v, psync::real_launch(), in, out, nvec, max_chunk_vecs, scale);
}
template <typename T, int TPB>
__global__ void __launch_bounds__(TPB)
    allreduce_sym_kernel(const __grid_constant__ ArenaView v, const __grid_constant__ SymPtrs p, int64_t nvec,
                         float scale) {
  allreduce_sym_body<T, TPB>(v, psync::real_launch(), p, nvec, scale);
}
template <typename T, int NR>
__global__ void __launch_bounds__(kTmaThreads)
    allreduce_sym_tma_kernel(const __grid_constant__ ArenaView v, const __grid_constant__ SymPtrs p, int64_t nvec,
                             float scale) {
  extern __shared__ __align__(128) unsigned char tma_smem[];
  allreduce_sym_tma_body<T, NR>(v, psync::real_launch(), p, nvec, scale, tma_smem);
}
// emulation: the grids of all ranks in one cooperative launch (rank count known at run time)
template <typename T>
__global__ void __launch_bounds__(kTmaThreads)
    allreduce_tma_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int64_t nvec, float scale) {
  extern __shared__ __align__(128) unsigned char tma_smem[];
  const EmuRank& e = ranks[blockIdx.x / blocks];
  const Launch L{(int)(blockIdx.x % blocks), blocks};
  SymPtrs p;
  for (int r = 0; r < kArenaMaxRanks; ++r) {
    p.in[r] = (const uint4*)e.sym_in[r];
    p.out[r] = (uint4*)e.sym_out[r];
  }
  switch (e.view.nranks) {
    case 2: allreduce_sym_tma_body<T, 2>(e.view, L, p, nvec, scale, tma_smem); break;
    case 4: allreduce_sym_tma_body<T, 4>(e.view, L, p, nvec, scale, tma_smem); break;
    case 8: allreduce_sym_tma_body<T, 8>(e.view, L, p, nvec, scale, tma_smem); break;
    default: break;  // the host side only launches it for 2, 4 or 8 ranks
  }
}

template <typename T, int NR>
void launch_sym_tma(const ArenaView& v, const SymPtrs& p, int64_t nvec, float scale, int grid, cudaStream_t stream) {
  static std::once_flag once;
  std::call_once(once, [] {
    BAGUA_CUDA_CHECK(cudaFuncSetAttribute(allreduce_sym_tma_kernel<T, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          TmaCfg<NR>::kSmemBytes));
  });
  allreduce_sym_tma_kernel<T, NR><<<grid, kTmaThreads, TmaCfg<NR>::kSmemBytes, stream>>>(v, p, nvec, scale);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    pair_average_kernel(const __grid_constant__ ArenaView v, const uint4* __restrict__ in, uint4* __restrict__ out,
                        int64_t nvec, int peer) {
  pair_average_body<T>(v, psync::real_launch(), in, out, nvec, peer);
}

// ---- emulation kernels: the grids of all ranks in one cooperative launch ------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    allreduce_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int mode, int64_t nvec, int64_t aux_vecs,
                         float scale) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  const Launch L{(int)(blockIdx.x % blocks), blocks};
  if (mode == (int)EmuAllreduceMode::OneShot) {
    allreduce_oneshot_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, nvec, aux_vecs, scale);
  } else if (mode == (int)EmuAllreduceMode::TwoShot) {
    allreduce_twoshot_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, nvec, aux_vecs, scale);
  } else {
    SymPtrs p;
    for (int r = 0; r < kArenaMaxRanks; ++r) {
      p.in[r] = (const uint4*)e.sym_in[r];
      p.out[r] = (uint4*)e.sym_out[r];
    }
    allreduce_sym_body<T>(e.view, L, p, nvec, scale);
  }
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    pair_average_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int64_t nvec, int symmetric) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  const Launch L{(int)(blockIdx.x % blocks), blocks};
  if (symmetric)
    pair_average_sym_body<T>(e.view, L, (const uint4*)e.in, (const uint4*)e.sym_in[e.peer], (uint4*)e.out, nvec, e.peer);
  else
    pair_average_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, nvec, e.peer);
}

__global__ void wait_probe_kernel(ArenaView v) {
  // waits for a phase signal from "rank 1" that nobody will ever send
  psync::cta_wait_phase(v, psync::real_launch(), 0, 1u << 1);
}

// Interference probe: occupies `grid` blocks of `threads` threads for `ns` nanoseconds of
// %globaltimer.  mode 0 only spins; mode 1 also streams over `buf` (reads and writes it back
// unchanged, 16 bytes per thread and iteration) for as long as it runs.  Bounded by the timer
// and by an iteration cap; touches nothing outside `buf`.
__global__ void occupy_kernel(uint4* buf, int64_t nvec, uint64_t ns, int mode) {
  const uint64_t t0 = psync::globaltimer_ns();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (uint64_t it = 0; it < (1ull << 26); ++it) {
    if (psync::globaltimer_ns() - t0 >= ns) break;
    if (mode == 1 && nvec > 0) {
      if (i >= nvec) i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
      if (i < nvec) {
        uint4 x = buf[i];
        buf[i] = x;
      }
      i += stride;
    } else {
      __nanosleep(100);
    }
  }
}

int pick_grid(const PeerArena& arena, size_t bytes, bool overlapped = false) {
  // one CTA per `bytes_per_cta` of payload, at least 1, at most the CTA budget: the arena's
  // for a call that has the GPU to itself, the (smaller) overlap budget for a bucket that is
  // reduced while backward kernels want the SMs
  const Tuning& t = Tuning::global();
  const int64_t per = std::max<int64_t>(t.bytes_per_cta.load(), 4096);
  int64_t cap = arena.max_blocks();
  if (overlapped) cap = std::min<int64_t>(cap, std::max<int64_t>(t.overlap_ctas.load(), 1));
  int64_t g = (int64_t)((bytes + per - 1) / per);
  g = std::max<int64_t>(1, std::min<int64_t>(g, cap));
  return (int)g;
}

template <typename T>
bool allreduce_t(PeerArena& arena, const void* in, void* out, int64_t n, float scale, cudaStream_t stream,
                 bool overlapped) {
  const size_t bytes = (size_t)n * sizeof(T);
  if (bytes == 0) return true;
  if (bytes % 16 != 0 || (uintptr_t)in % 16 != 0 || (uintptr_t)out % 16 != 0) return false;
  const int64_t nvec = (int64_t)(bytes / 16);
  const int N = arena.nranks();
  const Tuning& tune = Tuning::global();
  const int grid = pick_grid(arena, bytes, overlapped);
  // Buffers in the symmetric heap need no staging: above a small size (two signalling hops
  // instead of one) every rank reduces its own 1/N of the peers' buffers in place.  That moves
  // (N-1)/N·S per GPU and direction where the one-shot push moves (N-1)·S, also with two ranks.
  void *pin[kArenaMaxRanks], *pout[kArenaMaxRanks];
  const bool sym = arena.sym_translate(in, bytes, pin) && arena.sym_translate(out, bytes, pout);
  // One-shot through staging sends (N-1)·S per GPU in one hop, two-shot 2(N-1)/N·S in two hops:
  // with two ranks the wire bytes are equal, so one-shot always wins; otherwise it wins while
  // the extra bytes cost less than the extra hop (about 16 MB of wire traffic per GPU).
  const long oneshot_env = tune.oneshot_bytes.load();
  // (symmetric buffers: oneshot_sym_bytes; unset, 4 MB with two ranks, where the push sends no more
  // bytes than the pull and saves one signalling round, 128 KB otherwise)
  const long sym_env = tune.oneshot_sym_bytes.load();
  const size_t oneshot_max = sym                ? (sym_env >= 0 ? (size_t)sym_env : N == 2 ? ((size_t)4 << 20) : ((size_t)128 << 10))
                             : oneshot_env >= 0 ? (size_t)oneshot_env
                             : N == 2           ? ((size_t)512 << 20)
                                                : ((size_t)16 << 20) / (size_t)(N - 1);
  if (bytes <= oneshot_max) {
    arena.ensure_staging((size_t)N * bytes);
    ArenaView v = arena.next_view(grid, 0);
    allreduce_oneshot_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, nvec, nvec, scale);
  } else if (sym) {
    SymPtrs p;
    std::memset(&p, 0, sizeof(p));
    for (int r = 0; r < N; ++r) {
      p.in[r] = (const uint4*)pin[r];
      p.out[r] = (uint4*)pout[r];
    }
    // Large buckets: tiles travel through the bulk-copy engine (fused_allreduce_tma.cuh), which keeps
    // an order of magnitude more bytes in flight per SM, so a handful of blocks carries the link.
    const long tma_min = tune.tma_min_bytes.load();
    if (tma_min >= 0 && bytes >= (size_t)tma_min && (N == 2 || N == 4 || N == 8) &&
        (overlapped || tune.tma_isolated.load() != 0)) {
      const int64_t per = std::max<int64_t>(tune.tma_bytes_per_cta.load(), 64 << 10);
      int64_t cap = std::max<long>(overlapped ? tune.tma_overlap_ctas.load() : tune.tma_ctas.load(), 1);
      cap = std::min<int64_t>(cap, kArenaMaxBlocks);
      const int g2 = (int)std::max<int64_t>(1, std::min<int64_t>((int64_t)((bytes / N + per - 1) / per), cap));
      ArenaView v = arena.next_view(g2, 0);
      if (N == 2)
        launch_sym_tma<T, 2>(v, p, nvec, scale, g2, stream);
      else if (N == 4)
        launch_sym_tma<T, 4>(v, p, nvec, scale, g2, stream);
      else
        launch_sym_tma<T, 8>(v, p, nvec, scale, g2, stream);
      BAGUA_CUDA_CHECK(cudaGetLastError());
      arena.count_launch();
      return true;
    }
    // Narrower blocks (sym_threads = 128 or 256) spread the same number of threads over more SMs
    // and leave room on each for a compute kernel's blocks; the payload per block shrinks alike.
    const long tpb = tune.sym_threads.load();
    if (tpb == 128 || tpb == 256) {
      const int64_t per = std::max<int64_t>(tune.bytes_per_cta.load(), 4096) * tpb / kThreads;
      const int64_t cap = std::min<int64_t>(kArenaMaxBlocks, (int64_t)grid * (kThreads / tpb));
      const int g2 = (int)std::max<int64_t>(1, std::min<int64_t>((int64_t)((bytes + per - 1) / per), cap));
      ArenaView v = arena.next_view(g2, 0);
      if (tpb == 128)
        allreduce_sym_kernel<T, 128><<<g2, 128, 0, stream>>>(v, p, nvec, scale);
      else
        allreduce_sym_kernel<T, 256><<<g2, 256, 0, stream>>>(v, p, nvec, scale);
    } else {
      ArenaView v = arena.next_view(grid, 0);
      allreduce_sym_kernel<T, kThreads><<<grid, kThreads, 0, stream>>>(v, p, nvec, scale);
    }
  } else {
    const int64_t max_chunk = (nvec + N - 1) / N;
    arena.ensure_staging(((size_t)N * (size_t)max_chunk + (size_t)nvec) * 16);
    ArenaView v = arena.next_view(grid, 0);
    allreduce_twoshot_kernel<T>
        <<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, nvec, max_chunk, scale);
  }
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

template <typename T>
bool pair_average_t(PeerArena& arena, const void* in, void* out, int64_t n, int peer, cudaStream_t stream) {
  const size_t bytes = (size_t)n * sizeof(T);
  if (bytes == 0) return true;
  if (bytes % 16 != 0 || (uintptr_t)in % 16 != 0 || (uintptr_t)out % 16 != 0) return false;
  const int grid = pick_grid(arena, bytes);
  void* pin[kArenaMaxRanks];
  const long sym_min = Tuning::global().pair_sym_min_bytes.load();
  if (sym_min >= 0 && bytes >= (size_t)sym_min && arena.sym_translate(in, bytes, pin)) {
    // weights live in the symmetric heap on every rank: read the partner's copy directly (one pass over
    // the link instead of a push plus a local read; its second signalling round makes it the slower
    // choice for small buckets: 63 vs 55 us at 16 MB, 158 vs 199 us at 64 MB on two GPUs)
    ArenaView v = arena.next_view(grid, 0);
    pair_average_sym_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (const uint4*)pin[peer],
                                                               (uint4*)out, (int64_t)(bytes / 16), peer);
    BAGUA_CUDA_CHECK(cudaGetLastError());
    arena.count_launch();
    return true;
  }
  arena.ensure_staging(bytes);
  ArenaView v = arena.next_view(grid, 0);
  pair_average_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, (int64_t)(bytes / 16), peer);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

template <typename K, typename... Args>
void coop_launch(K kernel, int grid, Args... args) {
  int per_sm = 0, sms = 0, dev = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  void* argv[] = {(void*)&args...};
  BAGUA_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(kThreads), argv, 0, 0));
}

}  // namespace

Tuning& Tuning::global() {
  static Tuning t;
  static std::once_flag once;
  std::call_once(once, [] {
    t.oneshot_bytes = env_long("BAGUA_B200_ONESHOT_BYTES", -1);
    t.oneshot_sym_bytes = env_long("BAGUA_B200_ONESHOT_SYM_BYTES", -1);
    t.overlap_ctas = env_long("BAGUA_B200_OVERLAP_CTAS", 64);
    t.bytes_per_cta = env_long("BAGUA_B200_BYTES_PER_CTA", 64 << 10);
    t.nvls_overlap_ctas = env_long("BAGUA_B200_NVLS_OVERLAP_CTAS", 64);
    t.coop_overlap_ctas = env_long("BAGUA_B200_COOP_OVERLAP_CTAS", 32);
    t.sym_threads = env_long("BAGUA_B200_SYM_THREADS", 512);
    t.pair_sym_min_bytes = env_long("BAGUA_B200_PAIR_SYM_MIN_BYTES", 32 << 20);
    t.ce_min_bytes = env_long("BAGUA_B200_CE_MIN_BYTES", 8 << 20);
    t.ce_min_chunk_bytes = env_long("BAGUA_B200_CE_MIN_CHUNK_BYTES", 2 << 20);
    t.tma_min_bytes = env_long("BAGUA_B200_TMA_MIN_BYTES", 1 << 20);
    t.tma_isolated = env_long("BAGUA_B200_TMA_ISOLATED", 0);
    t.tma_ctas = env_long("BAGUA_B200_TMA_CTAS", 32);
    t.tma_overlap_ctas = env_long("BAGUA_B200_TMA_OVERLAP_CTAS", 16);
    t.tma_bytes_per_cta = env_long("BAGUA_B200_TMA_BYTES_PER_CTA", 256 << 10);
  });
  return t;
}

bool Tuning::set(const std::string& key, long value) {
  if (key == "oneshot_bytes") oneshot_bytes = value;
  else if (key == "oneshot_sym_bytes") oneshot_sym_bytes = value;
  else if (key == "overlap_ctas") overlap_ctas = value;
  else if (key == "bytes_per_cta") bytes_per_cta = value;
  else if (key == "nvls_overlap_ctas") nvls_overlap_ctas = value;
  else if (key == "coop_overlap_ctas") coop_overlap_ctas = value;
  else if (key == "sym_threads") sym_threads = value;
  else if (key == "pair_sym_min_bytes") pair_sym_min_bytes = value;
  else if (key == "ce_min_bytes") ce_min_bytes = value;
  else if (key == "ce_min_chunk_bytes") ce_min_chunk_bytes = value;
  else if (key == "tma_min_bytes") tma_min_bytes = value;
  else if (key == "tma_isolated") tma_isolated = value;
  else if (key == "tma_ctas") tma_ctas = value;
  else if (key == "tma_overlap_ctas") tma_overlap_ctas = value;
  else if (key == "tma_bytes_per_cta") tma_bytes_per_cta = value;
  else return false;
  return true;
}

std::vector<std::pair<std::string, long>> Tuning::items() const {
  return {{"oneshot_bytes", oneshot_bytes.load()},
          {"oneshot_sym_bytes", oneshot_sym_bytes.load()},
          {"overlap_ctas", overlap_ctas.load()},
          {"bytes_per_cta", bytes_per_cta.load()},
          {"nvls_overlap_ctas", nvls_overlap_ctas.load()},
          {"coop_overlap_ctas", coop_overlap_ctas.load()},
          {"sym_threads", sym_threads.load()},
          {"pair_sym_min_bytes", pair_sym_min_bytes.load()},
          {"ce_min_bytes", ce_min_bytes.load()},
          {"ce_min_chunk_bytes", ce_min_chunk_bytes.load()},
          {"tma_min_bytes", tma_min_bytes.load()},
          {"tma_isolated", tma_isolated.load()},
          {"tma_ctas", tma_ctas.load()},
          {"tma_overlap_ctas", tma_overlap_ctas.load()},
          {"tma_bytes_per_cta", tma_bytes_per_cta.load()}};
}

bool allreduce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, cudaStream_t stream,
               bool overlapped) {
  if (arena.nvls_enabled() && allreduce_nvls(arena, in, out, n, dt, scale, stream, overlapped)) return true;
  // Large symmetric buckets reduced under backward kernels: the copy engines carry the bytes
  // (fused_allreduce_ce.cu), the SMs only run two one-block sync kernels and a short reduction.
  const long ce_min = Tuning::global().ce_min_bytes.load();
  const long ce_chunk = std::max(0l, Tuning::global().ce_min_chunk_bytes.load());
  const size_t bytes = (size_t)n * dtype_bytes(dt);
  if (overlapped && ce_min >= 0 && bytes >= (size_t)ce_min && bytes / (size_t)arena.nranks() >= (size_t)ce_chunk &&
      allreduce_ce(arena, in, out, n, dt, scale, stream))
    return true;
  switch (dt) {
    case DType::F32: return allreduce_t<float>(arena, in, out, n, scale, stream, overlapped);
    case DType::F16: return allreduce_t<__half>(arena, in, out, n, scale, stream, overlapped);
    case DType::BF16: return allreduce_t<__nv_bfloat16>(arena, in, out, n, scale, stream, overlapped);
    default: return false;
  }
}

bool pair_average(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, int peer, cudaStream_t stream) {
  if (peer < 0 || peer >= arena.nranks() || peer == arena.rank()) return false;
  switch (dt) {
    case DType::F32: return pair_average_t<float>(arena, in, out, n, peer, stream);
    case DType::F16: return pair_average_t<__half>(arena, in, out, n, peer, stream);
    case DType::BF16: return pair_average_t<__nv_bfloat16>(arena, in, out, n, peer, stream);
    default: return false;
  }
}

void emu_launch_allreduce(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale,
                          EmuAllreduceMode mode, int64_t aux_vecs) {
  const int grid = nranks * blocks;
  const int m = (int)mode;
  switch (dt) {
    case DType::F32: coop_launch(allreduce_emu_kernel<float>, grid, dev, blocks, m, n * 4 / 16, aux_vecs, scale); break;
    case DType::F16: coop_launch(allreduce_emu_kernel<__half>, grid, dev, blocks, m, n * 2 / 16, aux_vecs, scale); break;
    case DType::BF16:
      coop_launch(allreduce_emu_kernel<__nv_bfloat16>, grid, dev, blocks, m, n * 2 / 16, aux_vecs, scale);
      break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated all-reduce: unsupported dtype");
  }
}

namespace {
template <typename T>
void emu_tma_t(const EmuRank* dev, int nranks, int blocks, int64_t nvec, float scale) {
  BAGUA_CHECK(nranks == 2 || nranks == 4 || nranks == 8, Communicator,
              "the bulk-copy all-reduce is built for 2, 4 or 8 ranks");
  const int smem = std::max(std::max((int)TmaCfg<2>::kSmemBytes, (int)TmaCfg<4>::kSmemBytes), (int)TmaCfg<8>::kSmemBytes);
  BAGUA_CUDA_CHECK(
      cudaFuncSetAttribute(allreduce_tma_emu_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 0, sms = 0, device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_tma_emu_kernel<T>, kTmaThreads, smem));
  const int grid = nranks * blocks;
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  void* args[] = {(void*)&dev, (void*)&blocks, (void*)&nvec, (void*)&scale};
  BAGUA_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)allreduce_tma_emu_kernel<T>, dim3(grid), dim3(kTmaThreads),
                                               args, (size_t)smem, 0));
}
}  // namespace

void emu_launch_allreduce_tma(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale) {
  switch (dt) {
    case DType::F32: emu_tma_t<float>(dev, nranks, blocks, n * 4 / 16, scale); break;
    case DType::F16: emu_tma_t<__half>(dev, nranks, blocks, n * 2 / 16, scale); break;
    case DType::BF16: emu_tma_t<__nv_bfloat16>(dev, nranks, blocks, n * 2 / 16, scale); break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated all-reduce: unsupported dtype");
  }
}

void emu_launch_pair_average(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, bool symmetric) {
  const int grid = nranks * blocks;
  const int sym = symmetric ? 1 : 0;
  switch (dt) {
    case DType::F32: coop_launch(pair_average_emu_kernel<float>, grid, dev, blocks, n * 4 / 16, sym); break;
    case DType::F16: coop_launch(pair_average_emu_kernel<__half>, grid, dev, blocks, n * 2 / 16, sym); break;
    case DType::BF16: coop_launch(pair_average_emu_kernel<__nv_bfloat16>, grid, dev, blocks, n * 2 / 16, sym); break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated pair average: unsupported dtype");
  }
}

void debug_occupy(void* buf, size_t bytes, int grid, int threads, double micros, int mode, cudaStream_t stream) {
  if (grid < 1 || threads < 32 || threads > 1024 || micros <= 0 || micros > 1e6) return;
  occupy_kernel<<<grid, threads, 0, stream>>>((uint4*)buf, (int64_t)(bytes / 16), (uint64_t)(micros * 1e3), mode);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

DeviceStatus debug_wait_timeout(int device, double wait_ms) {
  BAGUA_CUDA_CHECK(cudaSetDevice(device));
  uint32_t* pad = nullptr;
  DeviceStatus* host = nullptr;
  DeviceStatus* dev = nullptr;
  BAGUA_CUDA_CHECK(cudaMalloc((void**)&pad, kSigWords * sizeof(uint32_t)));
  BAGUA_CUDA_CHECK(cudaMemset(pad, 0, kSigWords * sizeof(uint32_t)));
  BAGUA_CUDA_CHECK(cudaHostAlloc((void**)&host, sizeof(DeviceStatus), cudaHostAllocMapped));
  std::memset(host, 0, sizeof(DeviceStatus));
  BAGUA_CUDA_CHECK(cudaHostGetDevicePointer((void**)&dev, host, 0));
  ArenaView v;
  std::memset(&v, 0, sizeof(v));
  v.signals[0] = pad;
  v.signals[1] = pad;  // never written
  v.status = dev;
  v.rank = 0;
  v.nranks = 2;
  v.epoch = 1;
  v.deadline_ns = (uint64_t)(wait_ms * 1e6);
  wait_probe_kernel<<<1, 32>>>(v);
  cudaError_t e = cudaDeviceSynchronize();
  DeviceStatus s;
  std::memcpy(&s, host, sizeof(s));
  cudaFree(pad);
  cudaFreeHost(host);
  BAGUA_CUDA_CHECK(e);
  return s;
}

}  // namespace fused
}  // namespace bagua
