// Device body of the fused ByteGrad kernel (see fused_bytegrad.cu for the algorithm).  Kept in
// a header so that the same source is compiled by nvcc into the sm_100a kernels and by the host
// compiler (-DBAGUA_HOST_EMULATION, host_emulation.h: a block is one warp of 32 OS threads)
// into tests/cpp/device_emulation.cc.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "minmax_device.cuh"
#include "peer_sync.cuh"

namespace bagua {
namespace fused {
namespace bytegrad_bodies {

using namespace kernels;
#ifdef BAGUA_HOST_EMULATION
constexpr int kThreads = 32;
#else
constexpr int kThreads = 512;
#endif
constexpr int kHdr = 32;

__device__ __forceinline__ uint32_t peers_mask(const ArenaView& v) {
  return ((1u << v.nranks) - 1u) & ~(1u << v.rank);
}

template <typename T>
__device__ __forceinline__ void write_header(uint8_t* slot, float mn, float mx) {
  T* h = reinterpret_cast<T*>(slot);
  same_value_store(h, mmdev::from_f<T>(mn));
  same_value_store(h + 1, mmdev::from_f<T>(mx));
}
template <typename T>
__device__ __forceinline__ mmdev::Grid read_grid(const uint8_t* slot) {
  const T* h = reinterpret_cast<const T*>(slot);
  return mmdev::make_grid(mmdev::to_f(same_value_load(h)), mmdev::to_f(same_value_load(h + 1)));
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

// `pipelined` changes how the reduced chunks travel back (the last two phases): instead of storing
// every 16 quantised bytes to all N ranks at once and waiting for all of them before dequantising
// anything, a rank quantises its chunk once into its own slot, copies it to one destination after
// the other — nearest successor first — and signals each destination as soon as that copy is
// complete; the receiver waits for one source at a time, in the order in which they finish, and
// dequantises a chunk while the next ones are still on the wire.  Same bytes, same values.
template <typename T>
__device__ __forceinline__ void bytegrad_body(const ArenaView& v, const psync::Launch& L, T* __restrict__ x,
                                              int64_t chunk, size_t slot_bytes, size_t scratch_off, float scale,
                                              bool pipelined = false) {
  const int me = v.rank, N = v.nranks, G = L.grid, b = L.block;
  const int64_t groups = chunk / 16;
  const int64_t lo = groups * b / G * 16, hi = groups * (b + 1) / G * 16;
  uint8_t* my_stage = v.staging[me];
  float2* part1 = reinterpret_cast<float2*>(my_stage + scratch_off);  // [N][G]
  float2* part2 = part1 + (size_t)N * G;                               // [G]
  const size_t ag_off = (size_t)N * slot_bytes;
  BAGUA_SHARED_ARRAY(mmdev::Grid, s_grid, kArenaMaxRanks, 5);
  BAGUA_SHARED_ARRAY(float, s_lut, kArenaMaxRanks * 256, 6);  // dequantiser tables, one per source chunk

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
    if (!pipelined) {
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
    } else {
      uint8_t* own = my_stage + ag_off + (size_t)me * slot_bytes + kHdr;
      for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
        float f[16];
        mmdev::load16(p + i, f);
        mmdev::store_q16(own + i, f, g);
      }
      // every thread copies the vectors it has just written itself, so no barrier is needed here
      for (int k = 1; k < N; ++k) {
        const int q = (me + k) % N;
        uint8_t* dst = v.staging[q] + ag_off + (size_t)me * slot_bytes + kHdr;
        for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16)
          *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(own + i);
        psync::cta_signal_phase(v, L, 1, 1u << q);
      }
    }
  }

  // ---- P5 ----
  // One chunk: quantised words -> table look-up -> 16-byte vectors of T, consecutive lanes on
  // consecutive vectors (a warp's store instruction covers 512 contiguous bytes).  This is the one
  // loop of the kernel that gains from the vector walk (the four-fold expansion makes it
  // store-bound); the others read 16 consecutive elements per thread, which measured faster.
  constexpr int VE = mmdev::Vec16<T>::VE;
  constexpr int U = 4;
  using QW = typename mmdev::QWord<VE>::type;
  const int64_t vhi = hi / VE, vfirst = lo / VE + threadIdx.x;
  auto expand = [&](const uint8_t* q, T* out, const float* lut) {
    for (int64_t i0 = vfirst; i0 < vhi; i0 += (int64_t)U * kThreads) {
      QW w[U] = {};
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * kThreads < vhi) w[u] = mmdev::load_qword<VE>(q, i0 + u * kThreads);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * kThreads >= vhi) continue;
        float f[VE];
        mmdev::lut_word(w[u], f, lut);
        mmdev::store_vec(out, i0 + u * kThreads, f);
      }
    }
  };
  if (ok && pipelined) {
    for (int k = 0; k < N; ++k) {
      const int c = (me - k + N) % N;  // own chunk, then the sources in the order in which they reach this rank
      if (k > 0) {
        ok = psync::cta_wait_phase(v, L, 1, 1u << c);
        if (!ok) break;
      }
      if (threadIdx.x == 0) s_grid[0] = read_grid<T>(my_stage + ag_off + (size_t)c * slot_bytes);
      __syncthreads();
      mmdev::build_dequant_lut<T>(s_lut, s_grid[0]);
      __syncthreads();
      expand(my_stage + ag_off + (size_t)c * slot_bytes + kHdr, x + (int64_t)c * chunk, s_lut);
      __syncthreads();  // the table is rebuilt for the next chunk
    }
  } else if (ok) {
    if (threadIdx.x < N) s_grid[threadIdx.x] = read_grid<T>(my_stage + ag_off + (size_t)threadIdx.x * slot_bytes);
    __syncthreads();
    for (int c = 0; c < N; ++c) mmdev::build_dequant_lut<T>(s_lut + c * 256, s_grid[c]);
    __syncthreads();
    for (int c = 0; c < N; ++c)
      expand(my_stage + ag_off + (size_t)c * slot_bytes + kHdr, x + (int64_t)c * chunk, s_lut + c * 256);
  }
  psync::cta_finish_op(v, L);
}

}  // namespace bytegrad_bodies
}  // namespace fused
}  // namespace bagua
