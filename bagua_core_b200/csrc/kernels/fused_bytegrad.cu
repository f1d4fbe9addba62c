// Fused ByteGrad: the whole MinMaxUInt8-compressed all-reduce of one bucket in ONE
// cooperative sm_100a kernel, exchanging compressed chunks by direct peer stores.
//
// Phases (block b of every rank owns the same 16-element groups of every chunk):
//   P1  partial min/max of my slice of each of the N chunks            → local scratch
//       ── grid barrier ──
//   P2  fold partials → grid per chunk; quantise my slice of chunk c and store it, with
//       the {min,max} header, straight into slot[me] of rank c's staging; signal c
//   P3  wait for the N-1 signals; dequantise the N slots of my chunk, sum in rank order
//       (fp32), scale, round to the tensor dtype into the bucket; partial min/max
//       ── grid barrier ──
//   P4  fold → grid; quantise the reduced slice once and store it into slot[me] of every
//       rank's all-gather area; signal everyone
//   P5  wait; dequantise slice b of all N chunks into the bucket
//
// HBM traffic ≈ 2 reads + 1 write of the bucket plus the 1-byte payloads; wire traffic is
// 2(N-1)/N · (S/4 + headers) per GPU.  The reference runs ≥ 40 launches and two NCCL
// collectives per bucket for the same result
// (bagua-core-internal/src/comm_ops/centralized_low_precision_synchronous.rs:16-73).
// Numerics follow the reference: values are rounded through the tensor dtype after every
// dequantise and after the reduction, headers are stored in the tensor dtype.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "fused.h"
#include "fused_emu.h"
#include "minmax_device.cuh"
#include "peer_sync.cuh"

namespace bagua {
namespace fused {

namespace {

using namespace kernels;
constexpr int kThreads = 512;
constexpr int kHdr = 32;

__device__ __forceinline__ uint32_t peers_mask(const ArenaView& v) {
  return ((1u << v.nranks) - 1u) & ~(1u << v.rank);
}

template <typename T>
__device__ __forceinline__ void write_header(uint8_t* slot, float mn, float mx) {
  T* h = reinterpret_cast<T*>(slot);
  h[0] = mmdev::from_f<T>(mn);
  h[1] = mmdev::from_f<T>(mx);
}
template <typename T>
__device__ __forceinline__ mmdev::Grid read_grid(const uint8_t* slot) {
  const T* h = reinterpret_cast<const T*>(slot);
  return mmdev::make_grid(mmdev::to_f(h[0]), mmdev::to_f(h[1]));
}
template <typename T>
__device__ __forceinline__ float round_through(float x) {
  return mmdev::to_f(mmdev::from_f<T>(x));
}

// Fold G partial {min,max} pairs; result valid in every thread.
__device__ __forceinline__ void fold_partials(const float2* part, int G, float& mn, float& mx) {
  mn = FLT_MAX;
  mx = -FLT_MAX;
  for (int i = threadIdx.x; i < G; i += kThreads) {
    const float2 p = part[i];
    mn = fminf(mn, p.x);
    mx = fmaxf(mx, p.y);
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (mn > mx) mn = mx = 0.f;
}

template <typename T>
__device__ __forceinline__ void bytegrad_body(const ArenaView& v, const psync::Launch& L, T* __restrict__ x,
                                              int64_t chunk, size_t slot_bytes, size_t scratch_off, float scale) {
  const int me = v.rank, N = v.nranks, G = L.grid, b = L.block;
  const int64_t groups = chunk / 16;
  const int64_t lo = groups * b / G * 16, hi = groups * (b + 1) / G * 16;
  uint8_t* my_stage = v.staging[me];
  float2* part1 = reinterpret_cast<float2*>(my_stage + scratch_off);  // [N][G]
  float2* part2 = part1 + (size_t)N * G;                               // [G]
  const size_t ag_off = (size_t)N * slot_bytes;
  __shared__ mmdev::Grid s_grid[kArenaMaxRanks];
  __shared__ float s_lut[kArenaMaxRanks * 256];  // dequantiser tables, one per source chunk

  bool ok = psync::cta_wait_prev_done(v, L);

  // ---- P1 ----
  if (ok) {
    for (int c = 0; c < N; ++c) {
      const T* p = x + (int64_t)c * chunk;
      float mn = FLT_MAX, mx = -FLT_MAX;
      for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
        float f[16];
        mmdev::load16(p + i, f);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          mn = fminf(mn, f[k]);
          mx = fmaxf(mx, f[k]);
        }
      }
      mmdev::block_minmax<kThreads>(mn, mx);
      if (threadIdx.x == 0) part1[(size_t)c * G + b] = make_float2(mn, mx);
    }
  }
  ok = psync::grid_barrier(v, L, 0) && ok;

  // ---- P2 ----
  if (ok) {
    for (int k = 1; k <= N; ++k) {
      const int c = (me + k) % N;  // peers first, own chunk last
      float mn, mx;
      fold_partials(part1 + (size_t)c * G, G, mn, mx);
      const mmdev::Grid g = mmdev::make_grid(round_through<T>(mn), round_through<T>(mx));
      uint8_t* slot = v.staging[c] + (size_t)me * slot_bytes;
      if (threadIdx.x == 0) write_header<T>(slot, mn, mx);  // every block writes the same header
      const T* p = x + (int64_t)c * chunk;
      uint8_t* q = slot + kHdr;
      for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
        float f[16];
        mmdev::load16(p + i, f);
        mmdev::store_q16(q + i, f, g);
      }
    }
    // one system-scope fence for all peers instead of N-1 serialised NVLink round trips
    psync::cta_signal_phase(v, L, 0, peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, peers_mask(v));
  }

  // ---- P3 ----
  float mn2 = FLT_MAX, mx2 = -FLT_MAX;
  if (ok) {
    if (threadIdx.x < N) s_grid[threadIdx.x] = read_grid<T>(my_stage + (size_t)threadIdx.x * slot_bytes);
    __syncthreads();
    for (int r = 0; r < N; ++r) mmdev::build_dequant_lut<T>(s_lut + r * 256, s_grid[r]);
    __syncthreads();
    T* out = x + (int64_t)me * chunk;
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float acc[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) acc[k] = 0.f;
      for (int r = 0; r < N; ++r) {
        float f[16];
        mmdev::lut_dq16(my_stage + (size_t)r * slot_bytes + kHdr + i, f, s_lut + r * 256);
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] += f[k];
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        acc[k] = round_through<T>(acc[k] * scale);
        mn2 = fminf(mn2, acc[k]);
        mx2 = fmaxf(mx2, acc[k]);
      }
      mmdev::store16(out + i, acc);
    }
  }
  mmdev::block_minmax<kThreads>(mn2, mx2);
  if (threadIdx.x == 0) part2[b] = make_float2(mn2, mx2);
  ok = psync::grid_barrier(v, L, 1) && ok;

  // ---- P4 ----
  if (ok) {
    float mn, mx;
    fold_partials(part2, G, mn, mx);
    const mmdev::Grid g = mmdev::make_grid(round_through<T>(mn), round_through<T>(mx));
    if (threadIdx.x < N) write_header<T>(v.staging[threadIdx.x] + ag_off + (size_t)me * slot_bytes, mn, mx);
    const T* p = x + (int64_t)me * chunk;
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float f[16];
      mmdev::load16(p + i, f);
      const uint4 packed = mmdev::pack_q16(f, g);
      for (int k = 0; k < N; ++k) {
        const int q = (me + k) % N;
        *reinterpret_cast<uint4*>(v.staging[q] + ag_off + (size_t)me * slot_bytes + kHdr + i) = packed;
      }
    }
    psync::cta_signal_phase(v, L, 1, peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, peers_mask(v));
  }

  // ---- P5 ----
  if (ok) {
    if (threadIdx.x < N) s_grid[threadIdx.x] = read_grid<T>(my_stage + ag_off + (size_t)threadIdx.x * slot_bytes);
    __syncthreads();
    for (int c = 0; c < N; ++c) mmdev::build_dequant_lut<T>(s_lut + c * 256, s_grid[c]);
    __syncthreads();
    for (int c = 0; c < N; ++c) {
      const uint8_t* q = my_stage + ag_off + (size_t)c * slot_bytes + kHdr;
      T* out = x + (int64_t)c * chunk;
      for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
        float f[16];
        mmdev::lut_dq16(q + i, f, s_lut + c * 256);
        mmdev::store16(out + i, f);
      }
    }
  }
  psync::cta_finish_op(v, L);
}

// one launch per rank
template <typename T>
__global__ void __launch_bounds__(kThreads)
    bytegrad_kernel(const __grid_constant__ ArenaView v, T* __restrict__ x, int64_t chunk, size_t slot_bytes,
                    size_t scratch_off, float scale) {
  bytegrad_body<T>(v, psync::real_launch(), x, chunk, slot_bytes, scratch_off, scale);
}

// single-GPU emulation: the grids of all ranks in one cooperative launch
template <typename T>
__global__ void __launch_bounds__(kThreads)
    bytegrad_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int64_t chunk, size_t slot_bytes,
                        size_t scratch_off, float scale) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  bytegrad_body<T>(e.view, psync::Launch{(int)(blockIdx.x % blocks), blocks}, (T*)e.in, chunk, slot_bytes, scratch_off,
                   scale);
}

template <typename T>
bool bytegrad_t(PeerArena& arena, void* bucket, int64_t n, bool average, cudaStream_t stream) {
  const int N = arena.nranks();
  if (n <= 0) return true;
  if (n % ((int64_t)16 * N) != 0 || (uintptr_t)bucket % 16 != 0) return false;
  const int64_t chunk = n / N;
  if ((chunk * (int64_t)sizeof(T)) % 16 != 0) return false;
  const size_t slot = (size_t)chunk + kHdr;
  // one CTA per 32 Ki elements of the bucket, up to the arena's limit for cooperative
  // kernels (one per SM by default: several HBM passes plus quantiser math per element)
  int64_t g = (n + (32 << 10) - 1) / (32 << 10);
  int grid = (int)std::max<int64_t>(1, std::min<int64_t>(g, arena.max_coop_blocks()));
  static int coop_limit = 0;
  if (coop_limit == 0) {
    int per_sm = 0, sms = 0, dev = 0;
    BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
    BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bytegrad_kernel<T>, kThreads, 0));
    coop_limit = std::max(1, per_sm * sms);
  }
  grid = std::min(grid, coop_limit);
  const size_t scratch_off = align_up(2 * (size_t)N * slot, 256);
  arena.ensure_staging(scratch_off + (size_t)(N + 1) * grid * sizeof(float2));
  ArenaView v = arena.next_view(grid, 2);
  T* x = (T*)bucket;
  int64_t chunk_arg = chunk;
  size_t slot_arg = slot, scratch_arg = scratch_off;
  float scale = average ? 1.0f / (float)N : 1.0f;
  void* args[] = {&v, &x, &chunk_arg, &slot_arg, &scratch_arg, &scale};
  BAGUA_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)bytegrad_kernel<T>, dim3(grid), dim3(kThreads), args, 0,
                                               stream));
  arena.count_launch();
  return true;
}

template <typename T>
void emu_bytegrad_t(const EmuRank* dev, int nranks, int blocks, int64_t n, float scale, size_t slot_bytes,
                    size_t scratch_off) {
  int per_sm = 0, sms = 0, device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bytegrad_emu_kernel<T>, kThreads, 0));
  const int grid = nranks * blocks;
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  int64_t chunk = n / nranks;
  void* args[] = {(void*)&dev, (void*)&blocks, (void*)&chunk, (void*)&slot_bytes, (void*)&scratch_off, (void*)&scale};
  BAGUA_CUDA_CHECK(
      cudaLaunchCooperativeKernel((const void*)bytegrad_emu_kernel<T>, dim3(grid), dim3(kThreads), args, 0, 0));
}

}  // namespace

void emu_launch_bytegrad(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale,
                         size_t slot_bytes, size_t scratch_off) {
  switch (dt) {
    case DType::F32: emu_bytegrad_t<float>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    case DType::F16: emu_bytegrad_t<__half>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    case DType::BF16: emu_bytegrad_t<__nv_bfloat16>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated ByteGrad: unsupported dtype");
  }
}

bool bytegrad(PeerArena& arena, void* bucket, int64_t n, DType dt, bool average, cudaStream_t stream) {
  switch (dt) {
    case DType::F32: return bytegrad_t<float>(arena, bucket, n, average, stream);
    case DType::F16: return bytegrad_t<__half>(arena, bucket, n, average, stream);
    case DType::BF16: return bytegrad_t<__nv_bfloat16>(arena, bucket, n, average, stream);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
