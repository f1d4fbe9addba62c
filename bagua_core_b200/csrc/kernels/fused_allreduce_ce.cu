// All-reduce on symmetric buffers whose bytes are moved by the GPU's copy engines, sm_100a.
//
// Why: a communication kernel that overlaps the backward pass costs the compute kernels
// (SMs it occupies) x (time it is resident), and on a step whose convolution kernels fill
// the GPU in whole waves, losing even a few SMs for the milliseconds a large bucket needs on
// the wire adds a wave to many of them (benchmarks/interference_probe.py).  The wire time
// cannot shrink, so for large buckets the transfer is taken off the SMs altogether:
//
//   sync kernel (1 block)   "my input is final" to every peer / wait for theirs
//   N-1 peer copies         rank r PULLS chunk r of every peer's input into local staging
//                           (cudaMemcpyAsync between device pointers: DMA over NVLink, no SM)
//   reduce kernel           chunk r = scale * sum over ranks, in rank order, fp32: a short
//                           HBM-bound burst of ordinary blocks that come and go
//   N-1 peer copies         rank r PUSHES the reduced chunk r into every peer's output
//   sync kernel (1 block)   "my copies are done" to every peer / wait for theirs
//
// all queued on the communicator's stream.  The two sync kernels are the only blocks that
// ever wait, and they are one block each.  In place is safe without a further round: chunk r
// of a peer's buffer is read only by rank r's own pulls, which precede its pushes on its
// stream.  Results are bit-identical to the load/store kernels (same order, same rounding).
// tests/cpp/device_emulation.cc replays this sequence with the same signalling calls under the
// thread sanitizer (in place and out of place).
//
// The reference has no counterpart (one NCCL call per bucket,
// bagua-core-internal/src/comm_ops/centralized_full_precision_synchronous.rs:16-55).
#include <cuda_runtime.h>

#include "../pool/resource_pool.h"
#include "fused.h"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {

namespace {

// One block: publish phase `phase` of this op to every peer and wait for theirs; the second
// one of an op also closes it (the `done` word that lets later ops reuse staging).
__global__ void ce_sync_kernel(const __grid_constant__ ArenaView v, int phase, int finish) {
  const psync::Launch L{0, 1};
  psync::cta_signal_phase(v, L, phase, all_peers_mask(v));
  psync::cta_wait_phase(v, L, phase, all_peers_mask(v));
  if (finish) psync::cta_finish_op(v, L);
}

// own[i] = scale * (sum over ranks r of (r == me ? own[i] : stage[r * slot_vecs + i])), r ascending.
template <typename T>
__global__ void __launch_bounds__(256)
    ce_reduce_kernel(uint4* own, const uint4* __restrict__ stage, int64_t cvec, int64_t slot_vecs, int nranks, int me,
                     float scale) {
  using O = VecOps<T>;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < cvec; i += (int64_t)gridDim.x * blockDim.x) {
    float a[O::N];
#pragma unroll
    for (int k = 0; k < O::N; ++k) a[k] = 0.f;
    for (int r = 0; r < nranks; ++r) O::acc(a, r == me ? own[i] : stage[(int64_t)r * slot_vecs + i]);
    own[i] = O::pack(a, scale);
  }
}

template <typename T>
bool allreduce_ce_t(PeerArena& arena, const void* in, void* out, int64_t n, float scale, cudaStream_t stream) {
  const size_t bytes = (size_t)n * sizeof(T);
  const int N = arena.nranks(), me = arena.rank();
  void *pin[kArenaMaxRanks], *pout[kArenaMaxRanks];
  if (bytes % 16 != 0 || (uintptr_t)in % 16 != 0 || (uintptr_t)out % 16 != 0) return false;
  if (!arena.sym_translate(in, bytes, pin) || !arena.sym_translate(out, bytes, pout)) return false;
  const int64_t nvec = (int64_t)(bytes / 16);
  auto c_lo = [&](int r) { return nvec * r / N; };
  const int64_t my_lo = c_lo(me), my_vecs = c_lo(me + 1) - my_lo;
  const int64_t slot_vecs = (nvec + N - 1) / N;
  // staging for the pulled chunks: this GPU's own memory, reused in stream order
  auto stage = MemoryPool::for_device(arena.device()).pull((size_t)N * (size_t)slot_vecs * 16, (uint64_t)stream);
  char* sp = (char*)stage->ptr();

  ArenaView v = arena.next_view(1, 0);
  ce_sync_kernel<<<1, 32, 0, stream>>>(v, 0, 0);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  if (my_vecs > 0) {
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(sp + (size_t)q * slot_vecs * 16, (const char*)pin[q] + (size_t)my_lo * 16,
                                       (size_t)my_vecs * 16, cudaMemcpyDeviceToDevice, stream));
    }
    // out-of-place: the reduction runs in the output buffer
    char* own = (char*)out + (size_t)my_lo * 16;
    if (out != in)
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(own, (const char*)in + (size_t)my_lo * 16, (size_t)my_vecs * 16,
                                       cudaMemcpyDeviceToDevice, stream));
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((my_vecs + 255) / 256, 148 * 8));
    ce_reduce_kernel<T><<<grid, 256, 0, stream>>>((uint4*)own, (const uint4*)sp, my_vecs, slot_vecs, N, me, scale);
    BAGUA_CUDA_CHECK(cudaGetLastError());
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      BAGUA_CUDA_CHECK(cudaMemcpyAsync((char*)pout[q] + (size_t)my_lo * 16, own, (size_t)my_vecs * 16,
                                       cudaMemcpyDeviceToDevice, stream));
    }
  }
  ce_sync_kernel<<<1, 32, 0, stream>>>(v, 1, 1);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

}  // namespace

bool allreduce_ce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, cudaStream_t stream) {
  switch (dt) {
    case DType::F32: return allreduce_ce_t<float>(arena, in, out, n, scale, stream);
    case DType::F16: return allreduce_ce_t<__half>(arena, in, out, n, scale, stream);
    case DType::BF16: return allreduce_ce_t<__nv_bfloat16>(arena, in, out, n, scale, stream);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
