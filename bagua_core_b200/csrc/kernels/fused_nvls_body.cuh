// Device body of the NVSwitch (multimem) all-reduce; see fused_nvls.cu for the algorithm.
// Kept in a header so that the same source is compiled by nvcc into the sm_100a kernel and by
// the host compiler (-DBAGUA_HOST_EMULATION) into tests/cpp/device_emulation.cc.  Under
// emulation the two switch primitives are modelled on a table of every rank's buffer: a
// multicast address is an address inside rank 0's buffer, `ld_reduce` adds the element at that
// offset over all ranks' buffers, `st` writes it into all of them.
#pragma once

#include <cuda_runtime.h>

#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {
namespace nvls_bodies {

using psync::Launch;

#ifdef BAGUA_HOST_EMULATION
// The emulated multicast object: every rank's mapping of the bound memory.
struct HostMulticast {
  char* base[kArenaMaxRanks] = {};
  int nranks = 0;
};
inline HostMulticast g_host_multicast;

template <typename T>
struct Multimem {
  static uint4 ld_reduce(const uint4* mc) {
    using O = VecOps<T>;
    const HostMulticast& m = g_host_multicast;
    const size_t off = (size_t)(reinterpret_cast<const char*>(mc) - m.base[0]);
    float a[O::N];
    for (int k = 0; k < O::N; ++k) a[k] = 0.f;
    for (int r = 0; r < m.nranks; ++r) O::acc(a, *reinterpret_cast<const uint4*>(m.base[r] + off));
    return O::pack(a, 1.0f);
  }
};
inline void multimem_st(uint4* mc, const uint4& x) {
  const HostMulticast& m = g_host_multicast;
  const size_t off = (size_t)(reinterpret_cast<char*>(mc) - m.base[0]);
  for (int r = 0; r < m.nranks; ++r) *reinterpret_cast<uint4*>(m.base[r] + off) = x;
}
#else
template <typename T>
struct Multimem;
template <>
struct Multimem<float> {
  __device__ static uint4 ld_reduce(const uint4* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
  }
};
template <>
struct Multimem<__half> {
  __device__ static uint4 ld_reduce(const uint4* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
  }
};
template <>
struct Multimem<__nv_bfloat16> {
  __device__ static uint4 ld_reduce(const uint4* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
  }
};

// The store is a 16-byte bit copy whatever the element type.
__device__ __forceinline__ void multimem_st(uint4* mc, const uint4& x) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(x.x), "r"(x.y), "r"(x.z),
               "r"(x.w)
               : "memory");
}
#endif

template <typename T>
__device__ __forceinline__ uint4 scaled(const uint4& x, float scale) {
  using O = VecOps<T>;
  float a[O::N];
#pragma unroll
  for (int k = 0; k < O::N; ++k) a[k] = 0.f;
  O::acc(a, x);
  return O::pack(a, scale);
}

// Rank r reduces chunk r through the switch and stores the result through the switch.
template <typename T>
__device__ __forceinline__ void allreduce_nvls_body(const ArenaView& v, const Launch& L, const uint4* mc_in,
                                                    uint4* mc_out, int64_t nvec, float scale) {
  const int me = v.rank, N = v.nranks;
  const int64_t c0 = nvec * me / N, len = nvec * (me + 1) / N - c0;
  const int64_t lo = c0 + len * L.block / L.grid, hi = c0 + len * (L.block + 1) / L.grid;
  const bool rescale = scale != 1.0f;

  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  bool ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  if (ok) {
    constexpr int U = 4;  // reductions in flight per thread
    int64_t i = lo + threadIdx.x;
    for (; i + (U - 1) * kThreads < hi; i += U * kThreads) {
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = Multimem<T>::ld_reduce(mc_in + i + u * kThreads);
#pragma unroll
      for (int u = 0; u < U; ++u) multimem_st(mc_out + i + u * kThreads, rescale ? scaled<T>(x[u], scale) : x[u]);
    }
    for (; i < hi; i += kThreads) {
      const uint4 x = Multimem<T>::ld_reduce(mc_in + i);
      multimem_st(mc_out + i, rescale ? scaled<T>(x, scale) : x);
    }
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

}  // namespace nvls_bodies
}  // namespace fused
}  // namespace bagua
