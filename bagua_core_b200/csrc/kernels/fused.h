// Host entry points of the fused communication kernels (sm_100a, peer stores over
// NVLink/NVSwitch through a PeerArena).  Each returns false — without launching
// anything — when the buffer layout is not eligible (alignment, size, dtype); the
// caller then takes the unfused library path.  All ranks of the communicator must make
// the same sequence of calls with the same sizes.
//
// What each call replaces in the reference (bagua-core-internal/src/comm_ops/):
//   allreduce      ncclAllReduce (+AVG), or alltoall → chunk reduce → allgather
//                  (centralized_full_precision_synchronous.rs:16-55)
//   bytegrad       min/max ×2N, compress, alltoall, decompress, chunk reduce, min/max,
//                  compress, allgather, decompress
//                  (centralized_low_precision_synchronous.rs:16-73)
//   pair_average   grouped send/recv with one peer + average kernel
//                  (decentralized_full_precision_synchronous.rs:62-92)
//   lp_ring        3 addmul, min/max, compress, 4 grouped send/recv, 3 decompress,
//                  3 add, copy (decentralized_low_precision_synchronous.rs:23-154)
#pragma once

#include <cuda_runtime_api.h>

#include <atomic>
#include <string>
#include <utility>
#include <vector>

#include "../comm/arena.h"
#include "../common.h"

namespace bagua {
namespace fused {

// Size thresholds and CTA budgets of the fused kernels.  Defaults come from the environment
// (BAGUA_B200_<KEY IN CAPITALS>); `set` changes them at run time for all later launches, which
// every rank must do alike (the thresholds select the algorithm, and ranks must agree on it).
struct Tuning {
  std::atomic<long> oneshot_bytes{-1};         // staging path: one-shot up to this size (-1: by rank count)
  std::atomic<long> oneshot_sym_bytes{-1};     // symmetric buffers: one-shot up to this size (-1: by rank count)
  std::atomic<long> overlap_ctas{64};          // CTA budget of a bucket reduced under backward kernels
  std::atomic<long> bytes_per_cta{64 << 10};   // payload per CTA below the budget
  std::atomic<long> nvls_overlap_ctas{64};     // the overlap budget of the multimem all-reduce
  std::atomic<long> coop_overlap_ctas{32};     // the overlap budget of the cooperative ByteGrad kernel
  std::atomic<long> sym_threads{512};          // threads per block of the symmetric all-reduce (128, 256 or 512)
  std::atomic<long> pair_sym_min_bytes{32 << 20};  // pair average: direct peer loads from this size on (-1: never)
  // symmetric buckets of at least this size, reduced under backward kernels, are moved by the copy
  // engines (allreduce_ce); -1: never
  std::atomic<long> ce_min_bytes{8 << 20};
  // ... and only when the chunk that travels between two ranks (size / ranks) is at least this large:
  // the path queues 2 (ranks - 1) copies per bucket, and below this size their issue cost on the
  // launching thread outweighs the SMs saved
  std::atomic<long> ce_min_chunk_bytes{2 << 20};
  // symmetric buffers of at least this size take the bulk-copy (TMA) all-reduce; -1: never
  std::atomic<long> tma_min_bytes{1 << 20};
  // 0: only buckets reduced under backward kernels take it (with the GPU to itself the load/store kernel
  // is as fast and SM count does not matter); 1: every eligible call
  std::atomic<long> tma_isolated{0};
  std::atomic<long> tma_ctas{32};              // its CTA budget when it has the GPU to itself
  std::atomic<long> tma_overlap_ctas{16};      // ... and under backward kernels
  std::atomic<long> tma_bytes_per_cta{256 << 10};  // bytes of the rank's own chunk per CTA below the budget
  static Tuning& global();
  bool set(const std::string& key, long value);  // false: unknown key
  std::vector<std::pair<std::string, long>> items() const;
};

// out = scale * sum_r in_r.  `in` and `out` may be the same buffer.  `overlapped`: the call runs
// while compute kernels want the SMs (a gradient bucket during backward), so it takes the
// overlap CTA budget instead of the arena's.
bool allreduce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, cudaStream_t stream,
               bool overlapped = false);

// The same through the NVSwitch's reduction units (multimem.ld_reduce / multimem.st); only for
// buffers inside a symmetric-heap slab that has a multicast mapping (BAGUA_B200_NVLS=1).
// `allreduce` tries this first.
bool allreduce_nvls(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale,
                    cudaStream_t stream, bool overlapped = false);

// The same for buffers in the symmetric heap with the bytes moved by the copy engines: rank r pulls
// chunk r of every peer's input (DMA), reduces it with a short local kernel and pushes the result
// into every peer's output (DMA); two one-block kernels do the signalling.  Returns false when the
// buffers are not symmetric.
bool allreduce_ce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, cudaStream_t stream);

// In-place ByteGrad on `bucket` (n elements, n % (16*nranks) == 0).
bool bytegrad(PeerArena& arena, void* bucket, int64_t n, DType dt, bool average, cudaStream_t stream,
              bool overlapped = false);

// out = (in + peer's in) / 2; `peer` pairs must be mutual.
bool pair_average(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, int peer, cudaStream_t stream);

// Low-precision ring gossip step on weights x with replicas w (own), l / r (neighbours').
bool lp_ring(PeerArena& arena, void* x, void* w, void* l, void* r, int64_t n, DType dt, cudaStream_t stream);

// ---- the communicator's own collectives over peer memory (fused_collectives.cu) -----------
// Chunks are `chunk_bytes` long (a multiple of 16, 16-byte aligned buffers).  The in-place
// forms of the library calls are accepted: all-gather with in == out + rank*chunk,
// all-to-all with in == out, reduce-scatter with out == in + rank*chunk.
// out[r] = rank r's `in`.
bool allgather(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, cudaStream_t stream);
// out[r] = chunk `rank` of rank r's `in`.
bool alltoall(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, cudaStream_t stream);
// All-to-all with per-pair sizes (counts and displacements in elements of `elem_bytes` bytes, one
// entry per rank, as in the library call).  Peer-memory form only for a send buffer in the
// symmetric heap — receivers pull their segments out of it —, which, like every symmetric
// allocation, all ranks decide alike; `in` and `out` must not overlap.
bool alltoall_v(PeerArena& arena, const void* in, size_t in_bytes, const int64_t* send_counts,
                const int64_t* send_displs, void* out, size_t out_bytes, const int64_t* recv_counts,
                const int64_t* recv_displs, size_t elem_bytes, cudaStream_t stream);
// out = scale * sum_r (chunk `rank` of rank r's `in`); f32 / f16 / bf16.
bool reduce_scatter(PeerArena& arena, const void* in, void* out, int64_t chunk_elems, DType dt, float scale,
                    cudaStream_t stream);
// buf on every rank = buf on `root`.
bool broadcast(PeerArena& arena, void* buf, size_t bytes, int root, cudaStream_t stream);
// Rank q's out = chunk q of root's `in` (in is only read on the root).
bool scatter(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int root, cudaStream_t stream);
// Root's out[r] = rank r's `in` (out is only written on the root).
bool gather(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int root, cudaStream_t stream);
// Root's out = scale * sum_r in_r; f32 / f16 / bf16.  `out` is only written on the root.
bool reduce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, int root,
            cudaStream_t stream);
// Returns (on the stream) once every rank's stream has reached the call.
bool barrier(PeerArena& arena, cudaStream_t stream);

// Interference probe (benchmarks/interference_probe.py): a kernel of `grid` x `threads` that stays
// resident for `micros` microseconds on `stream`; mode 1 also streams over [buf, buf + bytes).
void debug_occupy(void* buf, size_t bytes, int grid, int threads, double micros, int mode, cudaStream_t stream);

// Test hook: launches a one-CTA kernel that waits `wait_ms` for a signal nobody sends
// and returns the status record the host read back (code != 0 expected).  Uses only
// rank-local memory; needs no peers.
DeviceStatus debug_wait_timeout(int device, double wait_ms);

}  // namespace fused
}  // namespace bagua
