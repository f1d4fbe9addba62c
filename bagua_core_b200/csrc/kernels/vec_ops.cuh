// 16-byte vector helpers shared by the fused communication kernels: per-dtype fp32
// accumulation of a uint4 of elements, and the streaming block copy every kernel uses to
// move its slice to or from a peer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../comm/arena.h"
#include "host_emulation.h"

namespace bagua {
namespace fused {

#ifdef BAGUA_HOST_EMULATION
constexpr int kThreads = 32;  // OS threads per emulated block: one warp (thread t talks to rank t, so at least kArenaMaxRanks)
#else
constexpr int kThreads = 512;
#endif

template <typename T>
struct VecOps;
template <>
struct VecOps<float> {
  static constexpr int N = 4;
  __device__ static void acc(float (&a)[N], const uint4& r) {
    a[0] += __uint_as_float(r.x);
    a[1] += __uint_as_float(r.y);
    a[2] += __uint_as_float(r.z);
    a[3] += __uint_as_float(r.w);
  }
  __device__ static uint4 pack(const float (&a)[N], float s) {
    return make_uint4(__float_as_uint(a[0] * s), __float_as_uint(a[1] * s), __float_as_uint(a[2] * s),
                      __float_as_uint(a[3] * s));
  }
};
template <>
struct VecOps<__half> {
  static constexpr int N = 8;
  __device__ static void acc(float (&a)[N], const uint4& r) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __half22float2(h[k]);
      a[2 * k] += f.x;
      a[2 * k + 1] += f.y;
    }
  }
  __device__ static uint4 pack(const float (&a)[N], float s) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(a[2 * k] * s, a[2 * k + 1] * s);
    return r;
  }
};
template <>
struct VecOps<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void acc(float (&a)[N], const uint4& r) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      a[2 * k] += f.x;
      a[2 * k + 1] += f.y;
    }
  }
  __device__ static uint4 pack(const float (&a)[N], float s) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(a[2 * k] * s, a[2 * k + 1] * s);
    return r;
  }
};

__device__ __forceinline__ uint32_t all_peers_mask(const ArenaView& v) {
  return ((1u << v.nranks) - 1u) & ~(1u << v.rank);
}

// Streaming copy of vectors [lo, hi) from src to dst (same indexing), 4 in flight per thread.
__device__ __forceinline__ void copy_vecs(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t lo,
                                          int64_t hi) {
  int64_t i = lo + threadIdx.x;
  for (; i + 3 * kThreads < hi; i += 4 * kThreads) {
    uint4 a = src[i], b = src[i + kThreads], c = src[i + 2 * kThreads], d = src[i + 3 * kThreads];
    dst[i] = a;
    dst[i + kThreads] = b;
    dst[i + 2 * kThreads] = c;
    dst[i + 3 * kThreads] = d;
  }
  for (; i < hi; i += kThreads) dst[i] = src[i];
}

// One CTA per 64 KiB of payload, at least 1, at most `max_blocks`.
inline int grid_for_bytes(size_t bytes, int max_blocks) {
  int64_t g = (int64_t)((bytes + (64 << 10) - 1) / (64 << 10));
  g = g < 1 ? 1 : g;
  return (int)(g > max_blocks ? max_blocks : g);
}

}  // namespace fused
}  // namespace bagua
