// All-reduce (+scale) through the NVSwitch's multicast/reduction units (NVLS), sm_100a.
//
// For buckets that live in a symmetric-heap slab with a multicast mapping (comm/nvls.h).
// Rank r owns chunk r of the bucket: it issues `multimem.ld_reduce` on the multicast address
// of its chunk — the switch fetches that vector from all N GPUs, adds them and returns one
// result — scales it, and writes it back with `multimem.st`, which the switch stores into all
// N GPUs' memories.  Per GPU and direction S bytes cross NVLink instead of the 2(N-1)/N·S of
// the peer-to-peer two-shot, and no SM spends cycles on the additions.  The signalling is that
// of the symmetric two-shot kernel: "my input is final" before the loads, "my stores have
// been issued and fenced" after them; every rank receives the same bits because each vector
// is reduced once, by its owner.  Half types are accumulated in fp32 inside the switch
// (`.acc::f32`).
//
// Counterpart in the reference: the single ncclAllReduce of
// bagua-core-internal/src/comm_ops/centralized_full_precision_synchronous.rs:16-55 (NCCL
// picks its own NVLS algorithm when it can); this is the same idea inside the bucket kernel.
#include <cuda_runtime.h>

#include "fused.h"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {

namespace {

using psync::Launch;

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

template <typename T>
__device__ __forceinline__ uint4 scaled(const uint4& x, float scale) {
  using O = VecOps<T>;
  float a[O::N];
#pragma unroll
  for (int k = 0; k < O::N; ++k) a[k] = 0.f;
  O::acc(a, x);
  return O::pack(a, scale);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    allreduce_nvls_kernel(const __grid_constant__ ArenaView v, const uint4* mc_in, uint4* mc_out, int64_t nvec,
                          float scale) {
  const Launch L = psync::real_launch();
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

template <typename T>
bool allreduce_nvls_t(PeerArena& arena, const void* in, void* out, int64_t n, float scale, cudaStream_t stream) {
  const size_t bytes = (size_t)n * sizeof(T);
  static const size_t min_bytes = (size_t)env_long("BAGUA_B200_NVLS_MIN_BYTES", 256 << 10);
  if (bytes < min_bytes || bytes % 16 != 0 || (uintptr_t)in % 16 != 0 || (uintptr_t)out % 16 != 0) return false;
  const void* mc_in = arena.sym_multicast(in, bytes);
  void* mc_out = arena.sym_multicast(out, bytes);
  if (!mc_in || !mc_out) return false;
  const int grid = grid_for_bytes(bytes, arena.max_blocks());
  ArenaView v = arena.next_view(grid, 0);
  allreduce_nvls_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)mc_in, (uint4*)mc_out, (int64_t)(bytes / 16),
                                                          scale);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

}  // namespace

bool allreduce_nvls(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale,
                    cudaStream_t stream) {
  if (!arena.nvls_enabled()) return false;
  switch (dt) {
    case DType::F32: return allreduce_nvls_t<float>(arena, in, out, n, scale, stream);
    case DType::F16: return allreduce_nvls_t<__half>(arena, in, out, n, scale, stream);
    case DType::BF16: return allreduce_nvls_t<__nv_bfloat16>(arena, in, out, n, scale, stream);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
