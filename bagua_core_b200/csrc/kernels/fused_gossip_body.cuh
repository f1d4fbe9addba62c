// Device body of the fused low-precision ring gossip kernel (see fused_gossip.cu for the
// algorithm).  Kept in a header so that the same source is compiled by nvcc into the sm_100a
// kernels and by the host compiler (-DBAGUA_HOST_EMULATION, host_emulation.h: a block is one
// warp of 32 OS threads) into tests/cpp/device_emulation.cc.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "minmax_device.cuh"
#include "peer_sync.cuh"

namespace bagua {
namespace fused {
namespace gossip_bodies {

using namespace kernels;
#ifdef BAGUA_HOST_EMULATION
constexpr int kThreads = 32;
#else
constexpr int kThreads = 512;
#endif
constexpr int kHdr = 32;

template <typename T>
__device__ __forceinline__ float rt(float x) {
  return mmdev::to_f(mmdev::from_f<T>(x));
}

template <typename T>
__device__ __forceinline__ void lp_ring_body(const ArenaView& v, const psync::Launch& L, T* __restrict__ x,
                                             T* __restrict__ w, T* __restrict__ l, T* __restrict__ r, int64_t n,
                                             size_t slot_bytes, size_t scratch_off) {
  const int me = v.rank, N = v.nranks, G = L.grid, b = L.block;
  const int left = (me + N - 1) % N, right = (me + 1) % N;
  const uint32_t nb_mask = (1u << left) | (1u << right);
  const int64_t groups = n / 16;
  const int64_t lo = groups * b / G * 16, hi = groups * (b + 1) / G * 16;
  uint8_t* stage = v.staging[me];
  uint8_t* from_left = stage;                   // written by my left neighbour
  uint8_t* from_right = stage + slot_bytes;     // written by my right neighbour
  uint8_t* own = stage + 2 * slot_bytes;        // my own compressed difference
  float2* part = reinterpret_cast<float2*>(stage + scratch_off);
  const float third = 1.0f / 3.0f, m53 = -5.0f / 3.0f;
  BAGUA_SHARED_ARRAY(float, s_lut, 3 * 256, 6);  // dequantiser tables: left, right, own

  bool ok = psync::cta_wait_prev_done(v, L);

  // ---- P1: d = x + l/3 + r/3 - 5w/3 (stored in x), partial min/max ----
  float mn = FLT_MAX, mx = -FLT_MAX;
  if (ok) {
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float fx[16], fl[16], fr[16], fw[16];
      mmdev::load16(x + i, fx);
      mmdev::load16(l + i, fl);
      mmdev::load16(r + i, fr);
      mmdev::load16(w + i, fw);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        float d = rt<T>(fmaf(fl[k], third, fx[k]));
        d = rt<T>(fmaf(fr[k], third, d));
        d = rt<T>(fmaf(fw[k], m53, d));
        fx[k] = d;
        mn = fminf(mn, d);
        mx = fmaxf(mx, d);
      }
      mmdev::store16(x + i, fx);
    }
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (threadIdx.x == 0) part[b] = make_float2(mn, mx);
  ok = psync::grid_barrier(v, L, 0) && ok;

  // ---- P2: quantise d, store to both neighbours and to my own slot ----
  mmdev::Grid g_own;
  if (ok) {
    mn = FLT_MAX;
    mx = -FLT_MAX;
    for (int i = threadIdx.x; i < G; i += kThreads) {
      const float2 p = part[i];
      mn = fminf(mn, p.x);
      mx = fmaxf(mx, p.y);
    }
    mmdev::block_minmax<kThreads>(mn, mx);
    if (mn > mx) mn = mx = 0.f;
    g_own = mmdev::make_grid(rt<T>(mn), rt<T>(mx));
    uint8_t* to_left = v.staging[left] + slot_bytes;  // I am my left neighbour's right neighbour
    uint8_t* to_right = v.staging[right];             // ... and my right neighbour's left neighbour
    if (threadIdx.x == 0) {
      mmdev::store_header<T>(to_left, mn, mx);
      mmdev::store_header<T>(to_right, mn, mx);
      mmdev::store_header<T>(own, mn, mx);
    }
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float f[16];
      mmdev::load16(x + i, f);
      const uint4 packed = mmdev::pack_q16(f, g_own);
      *reinterpret_cast<uint4*>(to_left + kHdr + i) = packed;
      *reinterpret_cast<uint4*>(to_right + kHdr + i) = packed;
      *reinterpret_cast<uint4*>(own + kHdr + i) = packed;
    }
    psync::cta_signal_phase(v, L, 0, nb_mask);
    ok = psync::cta_wait_phase(v, L, 0, nb_mask);
  }

  // ---- P3: apply the three differences ----
  if (ok) {
    float a, c;
    mmdev::load_header<T>(from_left, a, c);
    const mmdev::Grid g_l = mmdev::make_grid(a, c);
    mmdev::load_header<T>(from_right, a, c);
    const mmdev::Grid g_r = mmdev::make_grid(a, c);
    mmdev::build_dequant_lut<T>(s_lut, g_l);
    mmdev::build_dequant_lut<T>(s_lut + 256, g_r);
    mmdev::build_dequant_lut<T>(s_lut + 512, g_own);
    __syncthreads();
    // This loop walks the slice as 16-byte vectors of T (VE elements), consecutive lanes on
    // consecutive vectors, with U vectors of every stream loaded before the first is used: its four
    // store streams then leave as contiguous 512-byte spans per warp instruction.  (The two loops
    // above read 16 consecutive elements per thread; the vector walk measured slower for them.)
    constexpr int VE = mmdev::Vec16<T>::VE;
    constexpr int U = 2;
    using QW = typename mmdev::QWord<VE>::type;
    const int64_t vhi = hi / VE, vfirst = lo / VE + threadIdx.x;
    constexpr int64_t kStep = (int64_t)U * kThreads;
    for (int64_t i0 = vfirst; i0 < vhi; i0 += kStep) {
      QW ql[U] = {}, qr[U] = {}, qo[U] = {};
      float cl[U][VE], cr[U][VE], cw[U][VE];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * kThreads < vhi) {
          ql[u] = mmdev::load_qword<VE>(from_left + kHdr, i0 + u * kThreads);
          qr[u] = mmdev::load_qword<VE>(from_right + kHdr, i0 + u * kThreads);
          qo[u] = mmdev::load_qword<VE>(own + kHdr, i0 + u * kThreads);
          mmdev::load_vec(l, i0 + u * kThreads, cl[u]);
          mmdev::load_vec(r, i0 + u * kThreads, cr[u]);
          mmdev::load_vec(w, i0 + u * kThreads, cw[u]);
        }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * kThreads >= vhi) continue;
        float d[VE];
        mmdev::lut_word(ql[u], d, s_lut);
#pragma unroll
        for (int k = 0; k < VE; ++k) cl[u][k] = cl[u][k] + d[k];
        mmdev::store_vec(l, i0 + u * kThreads, cl[u]);
        mmdev::lut_word(qr[u], d, s_lut + 256);
#pragma unroll
        for (int k = 0; k < VE; ++k) cr[u][k] = cr[u][k] + d[k];
        mmdev::store_vec(r, i0 + u * kThreads, cr[u]);
        mmdev::lut_word(qo[u], d, s_lut + 512);
#pragma unroll
        for (int k = 0; k < VE; ++k) cw[u][k] = rt<T>(d[k] + cw[u][k]);
        mmdev::store_vec(x, i0 + u * kThreads, cw[u]);
        mmdev::store_vec(w, i0 + u * kThreads, cw[u]);
      }
    }
  }
  psync::cta_finish_op(v, L);
}

}  // namespace gossip_bodies
}  // namespace fused
}  // namespace bagua
