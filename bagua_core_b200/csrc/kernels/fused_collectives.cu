// Peer-memory kernels for the communicator's own collectives (all-gather, all-to-all,
// reduce-scatter, broadcast, reduce, gather, scatter, barrier), sm_100a.  The reference forwards each of these to
// one library call (bagua-core-internal/src/communicators/mod.rs:560-1040); here each is one
// launch that moves the data with 16-byte stores over NVLink and synchronises with the
// arena's signal words, using the same block-b-pairs-with-block-b scheme as the fused
// all-reduce: block b of every rank owns slice b of every chunk.
//
//   exchange (all-gather, all-to-all)
//       through staging: my chunk for q → slot[me] of q's staging, signal, wait, copy the
//       N-1 slots out of my own staging;
//       symmetric output: my chunk for q → straight into q's output, between a "started"
//       and a "stores done" signal exchange (no staging copy).
//   reduce-scatter
//       through staging: chunk q of my input → slot[me] of q's staging, signal, wait, sum
//       the N contributions to chunk `me` in rank order (fp32 accumulation, rounded once);
//       symmetric input: chunk `me` of all N inputs is loaded directly.
//   broadcast
//       small: the root stores the buffer into every peer's staging;
//       large: scatter + all-gather, so that the root sends 2(N-1)/N·S instead of (N-1)·S:
//       the root stores chunk q into q's staging and its own chunk into everyone's, then
//       every other rank forwards the chunk it owns to the remaining ranks.
//   scatter / gather
//       the root stores chunk q into q's staging / everyone stores its chunk into the
//       root's staging; the receiving side copies out of its own staging.
//   reduce (to one rank)
//       small: everyone stores its input into the root's staging, the root sums in rank
//       order; large: reduce-scatter among all ranks, then every rank hands its reduced
//       chunk to the root (2(N-1)/N·S into the root instead of (N-1)·S).
//   all-to-all with per-pair sizes (send buffer in the symmetric heap)
//       every rank writes {offset, length} of each peer's segment into that peer's staging,
//       signals, and pulls its own segments directly out of the peers' send buffers; a second
//       signal exchange tells the senders that their buffers are no longer being read.
//   barrier
//       one CTA: signal every peer, wait for every peer.
#include <cuda_runtime.h>

#include "fused.h"
#include "fused_emu.h"
#include "fused_collectives_bodies.cuh"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {

namespace {

using psync::Launch;
using namespace collectives;

// ---- real kernels: one launch per rank ---------------------------------------------
__global__ void __launch_bounds__(kThreads)
    exchange_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t cvec, int src_stride,
                    int skip_local) {
  exchange_body(v, psync::real_launch(), in, out, cvec, src_stride, skip_local);
}
__global__ void __launch_bounds__(kThreads)
    exchange_sym_kernel(const __grid_constant__ ArenaView v, const uint4* in, const __grid_constant__ PeerPtrs out,
                        int64_t cvec, int src_stride, int skip_local) {
  exchange_sym_body(v, psync::real_launch(), in, out, cvec, src_stride, skip_local);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    reduce_scatter_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t cvec, float scale) {
  reduce_scatter_body<T>(v, psync::real_launch(), in, out, cvec, scale);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    reduce_scatter_sym_kernel(const __grid_constant__ ArenaView v, const __grid_constant__ ConstPeerPtrs in, uint4* out,
                              int64_t cvec, float scale) {
  reduce_scatter_sym_body<T>(v, psync::real_launch(), in, out, cvec, scale);
}
__global__ void __launch_bounds__(kThreads)
    broadcast_kernel(const __grid_constant__ ArenaView v, uint4* buf, int64_t nvec, int root, int two_phase) {
  if (two_phase)
    broadcast_twophase_body(v, psync::real_launch(), buf, nvec, root);
  else
    broadcast_direct_body(v, psync::real_launch(), buf, nvec, root);
}
__global__ void __launch_bounds__(kThreads)
    scatter_gather_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t cvec, int root,
                          int skip_local, int gather) {
  if (gather)
    gather_body(v, psync::real_launch(), in, out, cvec, root, skip_local);
  else
    scatter_body(v, psync::real_launch(), in, out, cvec, root, skip_local);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
    reduce_kernel(const __grid_constant__ ArenaView v, const uint4* in, uint4* out, int64_t nvec, int64_t max_chunk_vecs,
                  int root, float scale, int two_phase) {
  if (two_phase)
    reduce_twophase_body<T>(v, psync::real_launch(), in, out, nvec, max_chunk_vecs, root, scale);
  else
    reduce_direct_body<T>(v, psync::real_launch(), in, out, nvec, root, scale);
}
__global__ void __launch_bounds__(kThreads)
    alltoall_v_sym_kernel(const __grid_constant__ ArenaView v, const __grid_constant__ ConstBytePtrs in, uint8_t* out,
                          const __grid_constant__ VSegments seg) {
  alltoall_v_sym_body(v, psync::real_launch(), in, out, seg);
}
__global__ void __launch_bounds__(kThreads) barrier_kernel(const __grid_constant__ ArenaView v) {
  barrier_body(v, psync::real_launch());
}

// ---- emulation kernel: the grids of all ranks in one cooperative launch -------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    collective_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int kind, int64_t cvec, int aux, float scale) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  const Launch L{(int)(blockIdx.x % blocks), blocks};
  switch ((EmuCollective)kind) {
    case EmuCollective::AllGather:
    case EmuCollective::AllToAll: {
      const int stride = kind == (int)EmuCollective::AllToAll ? 1 : 0;
      const int skip_local = (aux >> 1) & 1;
      if (aux & 1) {
        PeerPtrs p;
        for (int r = 0; r < kArenaMaxRanks; ++r) p.p[r] = (uint4*)e.sym_out[r];
        exchange_sym_body(e.view, L, (const uint4*)e.in, p, cvec, stride, skip_local);
      } else {
        exchange_body(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, stride, skip_local);
      }
      break;
    }
    case EmuCollective::ReduceScatter:
      if (aux & 1) {
        ConstPeerPtrs p;
        for (int r = 0; r < kArenaMaxRanks; ++r) p.p[r] = (const uint4*)e.sym_in[r];
        reduce_scatter_sym_body<T>(e.view, L, p, (uint4*)e.out, cvec, scale);
      } else {
        reduce_scatter_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, scale);
      }
      break;
    case EmuCollective::BroadcastDirect: broadcast_direct_body(e.view, L, (uint4*)e.out, cvec, aux); break;
    case EmuCollective::BroadcastTwoPhase: broadcast_twophase_body(e.view, L, (uint4*)e.out, cvec, aux); break;
    case EmuCollective::Barrier: barrier_body(e.view, L); break;
    // aux = root | skip_local << 8 for the rooted collectives below
    case EmuCollective::Scatter:
      scatter_body(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, aux & 0xff, (aux >> 8) & 1);
      break;
    case EmuCollective::Gather:
      gather_body(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, aux & 0xff, (aux >> 8) & 1);
      break;
    case EmuCollective::ReduceDirect:
      reduce_direct_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, aux & 0xff, scale);
      break;
    case EmuCollective::ReduceTwoPhase:
      reduce_twophase_body<T>(e.view, L, (const uint4*)e.in, (uint4*)e.out, cvec, (cvec + e.view.nranks - 1) / e.view.nranks,
                              aux & 0xff, scale);
      break;
  }
}

__global__ void __launch_bounds__(kThreads)
    alltoall_v_emu_kernel(const EmuRank* __restrict__ ranks, const VSegments* __restrict__ segments, int blocks) {
  const int rank = (int)blockIdx.x / blocks;
  const EmuRank& e = ranks[rank];
  ConstBytePtrs p;
  for (int r = 0; r < kArenaMaxRanks; ++r) p.p[r] = (const uint8_t*)e.sym_in[r];
  alltoall_v_sym_body(e.view, Launch{(int)(blockIdx.x % blocks), blocks}, p, (uint8_t*)e.out, segments[rank]);
}

// Largest staging an exchange may ask for; bigger requests take the library path.
constexpr size_t kMaxStaging = (size_t)2 << 30;

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

bool exchange(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int src_stride, cudaStream_t stream) {
  const int N = arena.nranks(), me = arena.rank();
  if (chunk_bytes == 0) return true;
  if (chunk_bytes % 16 != 0 || !aligned16(in) || !aligned16(out)) return false;
  const int64_t cvec = (int64_t)(chunk_bytes / 16);
  const char* local_src = (const char*)in + (size_t)src_stride * me * chunk_bytes;
  const int skip_local = (local_src == (const char*)out + (size_t)me * chunk_bytes) ? 1 : 0;
  const bool in_place_a2a = src_stride == 1 && in == out;
  const int grid = grid_for_bytes(chunk_bytes * (size_t)N, arena.max_blocks());
  void* pout[kArenaMaxRanks];
  if (!in_place_a2a && chunk_bytes >= ((size_t)64 << 10) && arena.sym_translate(out, chunk_bytes * (size_t)N, pout)) {
    PeerPtrs p;
    std::memset(&p, 0, sizeof(p));
    for (int r = 0; r < N; ++r) p.p[r] = (uint4*)pout[r];
    ArenaView v = arena.next_view(grid, 0);
    exchange_sym_kernel<<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, p, cvec, src_stride, skip_local);
  } else {
    if (chunk_bytes * (size_t)N > kMaxStaging) return false;
    arena.ensure_staging(chunk_bytes * (size_t)N);
    ArenaView v = arena.next_view(grid, 0);
    exchange_kernel<<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, cvec, src_stride, skip_local);
  }
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

template <typename T>
bool reduce_scatter_t(PeerArena& arena, const void* in, void* out, int64_t chunk_elems, float scale,
                      cudaStream_t stream) {
  const int N = arena.nranks();
  const size_t chunk_bytes = (size_t)chunk_elems * sizeof(T);
  if (chunk_bytes == 0) return true;
  if (chunk_bytes % 16 != 0 || !aligned16(in) || !aligned16(out)) return false;
  const int64_t cvec = (int64_t)(chunk_bytes / 16);
  const int grid = grid_for_bytes(chunk_bytes * (size_t)N, arena.max_blocks());
  void* pin[kArenaMaxRanks];
  if (chunk_bytes >= ((size_t)64 << 10) && arena.sym_translate(in, chunk_bytes * (size_t)N, pin)) {
    ConstPeerPtrs p;
    std::memset(&p, 0, sizeof(p));
    for (int r = 0; r < N; ++r) p.p[r] = (const uint4*)pin[r];
    ArenaView v = arena.next_view(grid, 0);
    reduce_scatter_sym_kernel<T><<<grid, kThreads, 0, stream>>>(v, p, (uint4*)out, cvec, scale);
  } else {
    if (chunk_bytes * (size_t)N > kMaxStaging) return false;
    arena.ensure_staging(chunk_bytes * (size_t)N);
    ArenaView v = arena.next_view(grid, 0);
    reduce_scatter_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, cvec, scale);
  }
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

template <typename K, typename... Args>
void coop_launch_all_ranks(K kernel, int grid, Args... args) {
  int per_sm = 0, sms = 0, dev = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  void* argv[] = {(void*)&args...};
  BAGUA_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(kThreads), argv, 0, 0));
}

}  // namespace

bool allgather(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, cudaStream_t stream) {
  return exchange(arena, in, out, chunk_bytes, 0, stream);
}

bool alltoall(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, cudaStream_t stream) {
  return exchange(arena, in, out, chunk_bytes, 1, stream);
}

bool alltoall_v(PeerArena& arena, const void* in, size_t in_bytes, const int64_t* send_counts,
                const int64_t* send_displs, void* out, size_t out_bytes, const int64_t* recv_counts,
                const int64_t* recv_displs, size_t elem_bytes, cudaStream_t stream) {
  const int N = arena.nranks();
  if (in_bytes == 0 || elem_bytes == 0) return false;
  const char *a = (const char*)in, *b = (const char*)out;
  if (a < b + out_bytes && b < a + in_bytes) return false;  // overlapping buffers: library path
  void* pin[kArenaMaxRanks];
  if (!arena.sym_translate(in, in_bytes, pin)) return false;
  ConstBytePtrs p;
  VSegments seg;
  std::memset(&p, 0, sizeof(p));
  std::memset(&seg, 0, sizeof(seg));
  for (int r = 0; r < N; ++r) {
    p.p[r] = (const uint8_t*)pin[r];
    seg.send_off[r] = send_displs[r] * (int64_t)elem_bytes;
    seg.send_bytes[r] = send_counts[r] * (int64_t)elem_bytes;
    seg.recv_off[r] = recv_displs[r] * (int64_t)elem_bytes;
    seg.recv_bytes[r] = recv_counts[r] * (int64_t)elem_bytes;
    if (seg.send_off[r] < 0 || seg.send_bytes[r] < 0 || (size_t)(seg.send_off[r] + seg.send_bytes[r]) > in_bytes ||
        seg.recv_off[r] < 0 || seg.recv_bytes[r] < 0 || (size_t)(seg.recv_off[r] + seg.recv_bytes[r]) > out_bytes)
      throw BaguaError(ErrorKind::Communicator, "alltoall_v: a segment lies outside its tensor");
  }
  // Sizes differ from rank to rank, but block b of a rank pairs with block b of its peers: the
  // grid must not depend on them.
  const int grid = arena.max_blocks();
  arena.ensure_staging((size_t)N * 16);
  ArenaView v = arena.next_view(grid, 0);
  alltoall_v_sym_kernel<<<grid, kThreads, 0, stream>>>(v, p, (uint8_t*)out, seg);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

bool reduce_scatter(PeerArena& arena, const void* in, void* out, int64_t chunk_elems, DType dt, float scale,
                    cudaStream_t stream) {
  switch (dt) {
    case DType::F32: return reduce_scatter_t<float>(arena, in, out, chunk_elems, scale, stream);
    case DType::F16: return reduce_scatter_t<__half>(arena, in, out, chunk_elems, scale, stream);
    case DType::BF16: return reduce_scatter_t<__nv_bfloat16>(arena, in, out, chunk_elems, scale, stream);
    default: return false;
  }
}

bool broadcast(PeerArena& arena, void* buf, size_t bytes, int root, cudaStream_t stream) {
  const int N = arena.nranks();
  if (root < 0 || root >= N) return false;
  if (bytes == 0) return true;
  if (bytes % 16 != 0 || !aligned16(buf) || bytes > kMaxStaging) return false;
  const int64_t nvec = (int64_t)(bytes / 16);
  // Direct: the root sends (N-1)·S in one hop.  Two-phase: 2(N-1)/N·S per GPU in two hops.
  const int two_phase = (N > 2 && bytes * (size_t)(N - 1) > ((size_t)4 << 20)) ? 1 : 0;
  const int grid = grid_for_bytes(bytes, arena.max_blocks());
  arena.ensure_staging(bytes);
  ArenaView v = arena.next_view(grid, 0);
  broadcast_kernel<<<grid, kThreads, 0, stream>>>(v, (uint4*)buf, nvec, root, two_phase);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

namespace {

bool scatter_gather(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int root, bool gather,
                    cudaStream_t stream) {
  const int N = arena.nranks(), me = arena.rank();
  if (root < 0 || root >= N) return false;
  if (chunk_bytes == 0) return true;
  // Only the root's big buffer and every rank's chunk are touched; the root's pointers decide
  // alignment on the root, the chunk pointers elsewhere.
  const void* used_in = (gather || me == root) ? in : nullptr;
  void* used_out = (!gather || me == root) ? out : nullptr;
  if (chunk_bytes % 16 != 0 || !aligned16(used_in) || !aligned16(used_out)) return false;
  const size_t need = gather ? chunk_bytes * (size_t)N : chunk_bytes;
  if (need > kMaxStaging) return false;
  int skip_local = 0;
  if (me == root) {
    const char* big = gather ? (const char*)out : (const char*)in;
    const char* small = gather ? (const char*)in : (const char*)out;
    skip_local = (small == big + (size_t)me * chunk_bytes) ? 1 : 0;
  }
  const int grid = grid_for_bytes(chunk_bytes * (size_t)N, arena.max_blocks());
  arena.ensure_staging(need);
  ArenaView v = arena.next_view(grid, 0);
  scatter_gather_kernel<<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, (int64_t)(chunk_bytes / 16),
                                                       root, skip_local, gather ? 1 : 0);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

template <typename T>
bool reduce_t(PeerArena& arena, const void* in, void* out, int64_t n, int root, float scale, cudaStream_t stream) {
  const int N = arena.nranks(), me = arena.rank();
  const size_t bytes = (size_t)n * sizeof(T);
  if (bytes == 0) return true;
  if (bytes % 16 != 0 || !aligned16(in) || (me == root && !aligned16(out))) return false;
  const int64_t nvec = (int64_t)(bytes / 16);
  const int two_phase = (N > 2 && bytes * (size_t)(N - 1) > ((size_t)4 << 20)) ? 1 : 0;
  const int64_t max_chunk = (nvec + N - 1) / N;
  const size_t need = two_phase ? ((size_t)N * (size_t)max_chunk + (size_t)nvec) * 16 : (size_t)N * bytes;
  if (need > kMaxStaging) return false;
  const int grid = grid_for_bytes(bytes, arena.max_blocks());
  arena.ensure_staging(need);
  ArenaView v = arena.next_view(grid, 0);
  reduce_kernel<T><<<grid, kThreads, 0, stream>>>(v, (const uint4*)in, (uint4*)out, nvec, max_chunk, root, scale,
                                                  two_phase);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

}  // namespace

bool scatter(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int root, cudaStream_t stream) {
  return scatter_gather(arena, in, out, chunk_bytes, root, false, stream);
}

bool gather(PeerArena& arena, const void* in, void* out, size_t chunk_bytes, int root, cudaStream_t stream) {
  return scatter_gather(arena, in, out, chunk_bytes, root, true, stream);
}

bool reduce(PeerArena& arena, const void* in, void* out, int64_t n, DType dt, float scale, int root,
            cudaStream_t stream) {
  if (root < 0 || root >= arena.nranks()) return false;
  switch (dt) {
    case DType::F32: return reduce_t<float>(arena, in, out, n, root, scale, stream);
    case DType::F16: return reduce_t<__half>(arena, in, out, n, root, scale, stream);
    case DType::BF16: return reduce_t<__nv_bfloat16>(arena, in, out, n, root, scale, stream);
    default: return false;
  }
}

bool barrier(PeerArena& arena, cudaStream_t stream) {
  ArenaView v = arena.next_view(1, 0);
  barrier_kernel<<<1, kThreads, 0, stream>>>(v);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  arena.count_launch();
  return true;
}

void emu_launch_alltoall_v(const EmuRank* dev, const void* segments, int nranks, int blocks) {
  static_assert(sizeof(VSegments) == 4 * kArenaMaxRanks * sizeof(int64_t), "EmulatedArena::alltoall_v mirrors this layout");
  coop_launch_all_ranks(alltoall_v_emu_kernel, nranks * blocks, dev, (const VSegments*)segments, blocks);
}

void emu_launch_collective(const EmuRank* dev, int nranks, int blocks, EmuCollective kind, int64_t cvec, DType dt,
                           int aux, float scale) {
  const int grid = nranks * blocks;
  const int k = (int)kind;
  switch (dt) {
    case DType::F16: coop_launch_all_ranks(collective_emu_kernel<__half>, grid, dev, blocks, k, cvec, aux, scale); break;
    case DType::BF16:
      coop_launch_all_ranks(collective_emu_kernel<__nv_bfloat16>, grid, dev, blocks, k, cvec, aux, scale);
      break;
    default: coop_launch_all_ranks(collective_emu_kernel<float>, grid, dev, blocks, k, cvec, aux, scale); break;
  }
}

}  // namespace fused
}  // namespace bagua
