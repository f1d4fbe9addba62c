// Device helpers shared by the MinMaxUInt8 kernels and the fused communication kernels:
// dtype widening, 16-element group loads/stores, the quantiser and a block min/max.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "host_emulation.h"

namespace bagua {
namespace kernels {
namespace mmdev {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct Grid {
  float scale, lower, upper;
};

// scale = 255/(max-min+1e-7) evaluated as the reference does: float denominator,
// double division, rounded to float.
__device__ __forceinline__ Grid make_grid(float mn, float mx) {
  Grid g;
  const float denom = (mx - mn) + 1e-7f;
  g.scale = (float)(255.0 / (double)denom);
  g.upper = rintf(mx * g.scale);
  g.lower = g.upper - 255.0f;
  return g;
}

__device__ __forceinline__ uint8_t quantise(float x, const Grid& g) {
  float level = rintf(x * g.scale);
  level = fminf(level, g.upper);
  float r = level - g.lower;
  r = fminf(fmaxf(r, 0.f), 255.f);
  return (uint8_t)r;
}
__device__ __forceinline__ float dequantise(uint8_t q, const Grid& g) { return ((float)q + g.lower) / g.scale; }

// ---- chunk headers: {min, max} in the tensor dtype at the start of a compressed chunk.
// A chunk may start at any byte offset when chunk sizes are not multiples of 32 (the
// layout divides the buffer evenly), so unaligned headers go through byte copies.
template <typename T>
__device__ __forceinline__ void store_header(uint8_t* base, float mn, float mx) {
  T h[2] = {from_f<T>(mn), from_f<T>(mx)};
  if ((reinterpret_cast<uintptr_t>(base) % sizeof(T)) == 0) {
    same_value_store(reinterpret_cast<T*>(base), h[0]);
    same_value_store(reinterpret_cast<T*>(base) + 1, h[1]);
  } else {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(h);
#pragma unroll
    for (int i = 0; i < (int)(2 * sizeof(T)); ++i) base[i] = src[i];
  }
}
template <typename T>
__device__ __forceinline__ void load_header(const uint8_t* base, float& mn, float& mx) {
  T h[2];
  if ((reinterpret_cast<uintptr_t>(base) % sizeof(T)) == 0) {
    h[0] = same_value_load(reinterpret_cast<const T*>(base));
    h[1] = same_value_load(reinterpret_cast<const T*>(base) + 1);
  } else {
    uint8_t* dst = reinterpret_cast<uint8_t*>(h);
#pragma unroll
    for (int i = 0; i < (int)(2 * sizeof(T)); ++i) dst[i] = base[i];
  }
  mn = to_f(h[0]);
  mx = to_f(h[1]);
}

// ---- 16-element groups (p must be 16-byte aligned) --------------------------------
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float4 a = q[j];
    v[4 * j + 0] = a.x;
    v[4 * j + 1] = a.y;
    v[4 * j + 2] = a.z;
    v[4 * j + 3] = a.w;
  }
}
__device__ __forceinline__ void load16(const __half* p, float (&v)[16]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 a = q[j];
    const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __half22float2(h[k]);
      v[8 * j + 2 * k] = f.x;
      v[8 * j + 2 * k + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 a = q[j];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      v[8 * j + 2 * k] = f.x;
      v[8 * j + 2 * k + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void store16(float* p, const float (&v)[16]) {
  float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
  for (int j = 0; j < 4; ++j) q[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}
__device__ __forceinline__ void store16(__half* p, const float (&v)[16]) {
  uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 a;
    __half2* h = reinterpret_cast<__half2*>(&a);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(v[8 * j + 2 * k], v[8 * j + 2 * k + 1]);
    q[j] = a;
  }
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&v)[16]) {
  uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 a;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[8 * j + 2 * k], v[8 * j + 2 * k + 1]);
    q[j] = a;
  }
}

__device__ __forceinline__ uint4 pack_q16(const float (&v)[16], const Grid& g) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w[j] = (uint32_t)quantise(v[4 * j], g) | ((uint32_t)quantise(v[4 * j + 1], g) << 8) |
           ((uint32_t)quantise(v[4 * j + 2], g) << 16) | ((uint32_t)quantise(v[4 * j + 3], g) << 24);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store_q16(uint8_t* q, const float (&v)[16], const Grid& g) {
  *reinterpret_cast<uint4*>(q) = pack_q16(v, g);
}
__device__ __forceinline__ void unpack_dq16(const uint4& a, float (&v)[16], const Grid& g) {
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[4 * j + k] = dequantise((uint8_t)((w[j] >> (8 * k)) & 0xffu), g);
  }
}
__device__ __forceinline__ void load_dq16(const uint8_t* q, float (&v)[16], const Grid& g) {
  unpack_dq16(*reinterpret_cast<const uint4*>(q), v, g);
}

// ---- coalesced 16-byte vectors -------------------------------------------------------
// The fused kernels walk a slice as 16-byte vectors of T (VE = 4 floats or 8 halves) with
// consecutive lanes on consecutive vectors, so every load/store instruction of a warp
// covers one contiguous 512-byte span; the VE quantised bytes of a vector are stored as
// one 4- or 8-byte word at the same element offset.
template <typename T>
struct Vec16 {
  static constexpr int VE = 16 / (int)sizeof(T);
};
__device__ __forceinline__ void load_vec(const float* base, int64_t vec, float (&f)[4]) {
  const float4 a = reinterpret_cast<const float4*>(base)[vec];
  f[0] = a.x;
  f[1] = a.y;
  f[2] = a.z;
  f[3] = a.w;
}
__device__ __forceinline__ void load_vec(const __half* base, int64_t vec, float (&f)[8]) {
  const uint4 a = reinterpret_cast<const uint4*>(base)[vec];
  const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 v = __half22float2(h[k]);
    f[2 * k] = v.x;
    f[2 * k + 1] = v.y;
  }
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* base, int64_t vec, float (&f)[8]) {
  const uint4 a = reinterpret_cast<const uint4*>(base)[vec];
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 v = __bfloat1622float2(h[k]);
    f[2 * k] = v.x;
    f[2 * k + 1] = v.y;
  }
}
__device__ __forceinline__ void store_vec(float* base, int64_t vec, const float (&f)[4]) {
  reinterpret_cast<float4*>(base)[vec] = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void store_vec(__half* base, int64_t vec, const float (&f)[8]) {
  uint4 a;
  __half2* h = reinterpret_cast<__half2*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
  reinterpret_cast<uint4*>(base)[vec] = a;
}
__device__ __forceinline__ void store_vec(__nv_bfloat16* base, int64_t vec, const float (&f)[8]) {
  uint4 a;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  reinterpret_cast<uint4*>(base)[vec] = a;
}
// quantised bytes of vector `vec` (payload pointer q must be 8-byte aligned)
__device__ __forceinline__ uint32_t pack_q4(const float* f, const Grid& g) {
  return (uint32_t)quantise(f[0], g) | ((uint32_t)quantise(f[1], g) << 8) | ((uint32_t)quantise(f[2], g) << 16) |
         ((uint32_t)quantise(f[3], g) << 24);
}
__device__ __forceinline__ uint32_t pack_qvec(const float (&f)[4], const Grid& g) { return pack_q4(f, g); }
__device__ __forceinline__ uint2 pack_qvec(const float (&f)[8], const Grid& g) {
  return make_uint2(pack_q4(f, g), pack_q4(f + 4, g));
}
__device__ __forceinline__ void store_qword(uint8_t* q, int64_t vec, uint32_t w) {
  reinterpret_cast<uint32_t*>(q)[vec] = w;
}
__device__ __forceinline__ void store_qword(uint8_t* q, int64_t vec, uint2 w) { reinterpret_cast<uint2*>(q)[vec] = w; }
// the quantised word of one vector: loaded first (so that several can be in flight), looked up later
template <int VE>
struct QWord;
template <>
struct QWord<4> {
  using type = uint32_t;
};
template <>
struct QWord<8> {
  using type = uint2;
};
template <int VE>
__device__ __forceinline__ typename QWord<VE>::type load_qword(const uint8_t* q, int64_t vec) {
  return reinterpret_cast<const typename QWord<VE>::type*>(q)[vec];
}
__device__ __forceinline__ void lut_word(uint32_t w, float (&f)[4], const float* lut) {
#pragma unroll
  for (int k = 0; k < 4; ++k) f[k] = lut[(w >> (8 * k)) & 0xffu];
}
__device__ __forceinline__ void lut_word(uint2 w, float (&f)[8], const float* lut) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[k] = lut[(w.x >> (8 * k)) & 0xffu];
    f[4 + k] = lut[(w.y >> (8 * k)) & 0xffu];
  }
}
__device__ __forceinline__ void lut_dqvec(const uint8_t* q, int64_t vec, float (&f)[4], const float* lut) {
  lut_word(load_qword<4>(q, vec), f, lut);
}
__device__ __forceinline__ void lut_dqvec(const uint8_t* q, int64_t vec, float (&f)[8], const float* lut) {
  lut_word(load_qword<8>(q, vec), f, lut);
}

// A chunk's dequantiser only has 256 possible outputs: tabulate them once per block (with
// the exact IEEE division, and the rounding through the tensor dtype that a store would
// apply) and turn every element into one shared-memory lookup.  Caller syncs the block.
template <typename T>
__device__ __forceinline__ void build_dequant_lut(float* lut, const Grid& g) {
  for (int q = threadIdx.x; q < 256; q += blockDim.x) lut[q] = to_f(from_f<T>(dequantise((uint8_t)q, g)));
}
__device__ __forceinline__ void lut_dq16(const uint8_t* q, float (&v)[16], const float* lut) {
  const uint4 a = *reinterpret_cast<const uint4*>(q);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int k = 0; k < 4; ++k) v[4 * j + k] = lut[(w[j] >> (8 * k)) & 0xffu];
  }
}

// Block-wide min/max; the result is valid in every thread.
template <int kThreads>
__device__ __forceinline__ void block_minmax(float& mn, float& mx) {
  BAGUA_SHARED_ARRAY(float, s_mn, kThreads / 32, 2);
  BAGUA_SHARED_ARRAY(float, s_mx, kThreads / 32, 3);
  BAGUA_SHARED_ARRAY(float, s_out, 2, 4);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protects s_* against a previous call's readers
  if (lane == 0) {
    s_mn[warp] = mn;
    s_mx[warp] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    float a = lane < kThreads / 32 ? s_mn[lane] : 3.402823466e+38f;
    float b = lane < kThreads / 32 ? s_mx[lane] : -3.402823466e+38f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a = fminf(a, __shfl_xor_sync(0xffffffffu, a, o));
      b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    if (lane == 0) {
      s_out[0] = a;
      s_out[1] = b;
    }
  }
  __syncthreads();
  mn = s_out[0];
  mx = s_out[1];
}

}  // namespace mmdev
}  // namespace kernels
}  // namespace bagua
