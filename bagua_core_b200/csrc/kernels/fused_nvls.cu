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
#include "fused_nvls_body.cuh"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {

namespace {

using psync::Launch;
using namespace nvls_bodies;

template <typename T>
__global__ void __launch_bounds__(kThreads)
    allreduce_nvls_kernel(const __grid_constant__ ArenaView v, const uint4* mc_in, uint4* mc_out, int64_t nvec,
                          float scale) {
  allreduce_nvls_body<T>(v, psync::real_launch(), mc_in, mc_out, nvec, scale);
}

template <typename T>
bool allreduce_nvls_t(PeerArena& arena, const void* in, void* out, int64_t n, float scale, cudaStream_t stream,
                      bool overlapped) {
  const size_t bytes = (size_t)n * sizeof(T);
  static const size_t min_bytes = (size_t)env_long("BAGUA_B200_NVLS_MIN_BYTES", 256 << 10);
  if (bytes < min_bytes || bytes % 16 != 0 || (uintptr_t)in % 16 != 0 || (uintptr_t)out % 16 != 0) return false;
  const void* mc_in = arena.sym_multicast(in, bytes);
  void* mc_out = arena.sym_multicast(out, bytes);
  if (!mc_in || !mc_out) return false;
  // The switch does the additions and the fan-out, so an SM issues one load and one store per
  // 16 bytes of its chunk whatever the rank count: a bucket reduced under backward kernels gets
  // by with the small overlap budget.
  const Tuning& t = Tuning::global();
  int cap = arena.max_blocks();
  if (overlapped) cap = (int)std::min<long>(cap, std::max<long>(t.nvls_overlap_ctas.load(), 1));
  const int grid = grid_for_bytes(bytes, cap);
  ArenaView v = arena.next_view(grid, 0);
  allreduce_nvls_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)mc_in, (uint4*)mc_out, (int64_t)(bytes / 16),
                                                          scale);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

}  // namespace

bool allreduce_nvls(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale,
                    cudaStream_t stream, bool overlapped) {
  if (!arena.nvls_enabled()) return false;
  switch (dt) {
    case DType::F32: return allreduce_nvls_t<float>(arena, in, out, n, scale, stream, overlapped);
    case DType::F16: return allreduce_nvls_t<__half>(arena, in, out, n, scale, stream, overlapped);
    case DType::BF16: return allreduce_nvls_t<__nv_bfloat16>(arena, in, out, n, scale, stream, overlapped);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
