// Device bodies of the fused all-reduce and pair-average kernels (see fused_allreduce.cu for
// the algorithms).  Kept in a header so that the same source is compiled twice: by nvcc into
// the sm_100a kernels, and by the host compiler (-DBAGUA_HOST_EMULATION, host_emulation.h)
// into the thread-per-CUDA-thread program tests/cpp/device_emulation.cc, which runs them
// under ThreadSanitizer together with the collective kernels' bodies.
#pragma once

#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {
namespace allreduce_bodies {

using psync::Launch;

// ---------------------------------------------------------------------------------
// one-shot
// ---------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void allreduce_oneshot_body(const ArenaView& v, const Launch& L,
                                                       const uint4* in, uint4* out,  // may be the same buffer
                                                       int64_t nvec, int64_t slot_vecs, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  const int64_t lo = nvec * L.block / L.grid, hi = nvec * (L.block + 1) / L.grid;
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      uint4* dst = reinterpret_cast<uint4*>(v.staging[q]) + (int64_t)me * slot_vecs;
      copy_vecs(dst, in, lo, hi);
    }
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) {
        const uint4 x = (r == me) ? in[i] : mine[(int64_t)r * slot_vecs + i];
        O::acc(a, x);
      }
      out[i] = O::pack(a, scale);
    }
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// two-shot through staging
// ---------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void allreduce_twoshot_body(const ArenaView& v, const Launch& L,
                                                       const uint4* in, uint4* out,  // may be the same buffer
                                                       int64_t nvec, int64_t max_chunk_vecs, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  const int G = L.grid, b = L.block;
  auto chunk_lo = [&](int c) { return nvec * c / N; };
  // block slice inside chunk c
  auto slice = [&](int c, int64_t& lo, int64_t& hi) {
    const int64_t c0 = chunk_lo(c), len = chunk_lo(c + 1) - c0;
    lo = c0 + len * b / G;
    hi = c0 + len * (b + 1) / G;
  };
  const int64_t ag_base = (int64_t)N * max_chunk_vecs;  // all-gather area follows the N reduce-scatter slots

  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    // step A: push my slice of chunk q into slot[me] of q
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      int64_t lo, hi;
      slice(q, lo, hi);
      uint4* dst = reinterpret_cast<uint4*>(v.staging[q]) + (int64_t)me * max_chunk_vecs - chunk_lo(q);
      copy_vecs(dst, in, lo, hi);
    }
    // one fence for all peers: a system-scope fence waits for every outstanding remote
    // store, so fencing per peer would serialise N-1 NVLink round trips
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    // step B: reduce my chunk in rank order, scale, store locally and to every peer
    int64_t lo, hi;
    slice(me, lo, hi);
    const int64_t c0 = chunk_lo(me);
    const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) {
        const uint4 x = (r == me) ? in[i] : mine[(int64_t)r * max_chunk_vecs + (i - c0)];
        O::acc(a, x);
      }
      const uint4 res = O::pack(a, scale);
      out[i] = res;
      for (int k = 1; k < N; ++k) {
        const int q = (me + k) % N;
        reinterpret_cast<uint4*>(v.staging[q])[ag_base + i] = res;
      }
    }
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  if (ok) {
    // step C: collect the other chunks from my own all-gather area
    const uint4* ag = reinterpret_cast<const uint4*>(v.staging[me]) + ag_base;
    for (int k = 1; k < N; ++k) {
      const int q = (me + k) % N;
      int64_t lo, hi;
      slice(q, lo, hi);
      copy_vecs(out, ag, lo, hi);
    }
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// two-shot on symmetric buffers: no staging at all
// ---------------------------------------------------------------------------------
// `in` and `out` live in the symmetric heap, so every rank can address every rank's copy.
// Rank r owns chunk r: it loads chunk r of all N inputs (N-1 of them over NVLink), sums in
// rank order, scales, and stores the result into chunk r of all N outputs.  Two signalling
// exchanges: "my input is ready" before the loads, "my stores are done" after them.  Wire
// per GPU: (N-1)/N·S in, (N-1)/N·S out; HBM traffic is the bucket itself, once.
struct SymPtrs {
  const uint4* in[kArenaMaxRanks];
  uint4* out[kArenaMaxRanks];
};

// NR is the rank count when it is 2, 4 or 8 (the loops over ranks then unroll with no
// predicates and U = 16 / NR vectors per thread keep 16 loads in flight whatever the rank
// count), 0 for any other count (bound checks against v.nranks, U = 2).
// TPB = threads per block of the launch (kThreads in the emulation).
template <typename T, int NR, int TPB = kThreads>
__device__ __forceinline__ void allreduce_sym_body_n(const ArenaView& v, const Launch& L, const SymPtrs& p,
                                                     int64_t nvec, float scale) {
  using O = VecOps<T>;
  constexpr int kThreads = TPB;  // shadows the file-wide constant inside this body
  constexpr int R = NR > 0 ? NR : kArenaMaxRanks;  // unrolled extent of the rank loops
  constexpr int U = NR > 0 ? 16 / NR : 2;          // vectors per thread per iteration
  const int me = v.rank, N = NR > 0 ? NR : v.nranks;
  const int G = L.grid, b = L.block;
  const int64_t c0 = nvec * me / N, len = nvec * (me + 1) / N - c0;
  const int64_t lo = c0 + len * b / G, hi = c0 + len * (b + 1) / G;

  // first signal: every peer's block b has started, i.e. that peer's input is final
  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  bool ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  if (ok) {
    int64_t i = lo + threadIdx.x;
    for (; i + (U - 1) * kThreads < hi; i += U * kThreads) {
      uint4 x[U][R];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r < N) x[u][r] = p.in[r][i + u * kThreads];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float a[O::N];
#pragma unroll
        for (int k = 0; k < O::N; ++k) a[k] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r < N) O::acc(a, x[u][r]);
        const uint4 res = O::pack(a, scale);
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r < N) p.out[r][i + u * kThreads] = res;
      }
    }
    for (; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) O::acc(a, p.in[r][i]);
      const uint4 res = O::pack(a, scale);
      for (int r = 0; r < N; ++r) p.out[r][i] = res;
    }
    // second signal: my stores into everyone's output are complete / theirs into mine
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

template <typename T, int TPB = kThreads>
__device__ __forceinline__ void allreduce_sym_body(const ArenaView& v, const Launch& L, const SymPtrs& p,
                                                   int64_t nvec, float scale) {
  switch (v.nranks) {
    case 2: allreduce_sym_body_n<T, 2, TPB>(v, L, p, nvec, scale); break;
    case 4: allreduce_sym_body_n<T, 4, TPB>(v, L, p, nvec, scale); break;
    case 8: allreduce_sym_body_n<T, 8, TPB>(v, L, p, nvec, scale); break;
    default: allreduce_sym_body_n<T, 0, TPB>(v, L, p, nvec, scale); break;
  }
}

// ---------------------------------------------------------------------------------
// pair average: out = (in + peer's in) / 2
// ---------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void pair_average_body(const ArenaView& v, const Launch& L, const uint4* __restrict__ in,
                                                  uint4* __restrict__ out, int64_t nvec, int peer) {
  using O = VecOps<T>;
  const int64_t lo = nvec * L.block / L.grid, hi = nvec * (L.block + 1) / L.grid;
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    copy_vecs(reinterpret_cast<uint4*>(v.staging[peer]), in, lo, hi);
    psync::cta_signal_phase(v, L, 0, 1u << peer);
    ok = psync::cta_wait_phase(v, L, 0, 1u << peer);
  }
  if (ok) {
    const uint4* got = reinterpret_cast<const uint4*>(v.staging[v.rank]);
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      O::acc(a, in[i]);
      O::acc(a, got[i]);
      out[i] = O::pack(a, 0.5f);
    }
  }
  psync::cta_finish_op(v, L);
}

// Pair average on symmetric buffers: the partner's weights are loaded straight from its
// memory (no staging copy).  First signal: both sides have started, so both inputs are final;
// second signal: both sides are done reading, so either may overwrite its weights again.
template <typename T>
__device__ __forceinline__ void pair_average_sym_body(const ArenaView& v, const Launch& L,
                                                      const uint4* __restrict__ in,
                                                      const uint4* __restrict__ peer_in, uint4* __restrict__ out,
                                                      int64_t nvec, int peer) {
  using O = VecOps<T>;
  const int64_t lo = nvec * L.block / L.grid, hi = nvec * (L.block + 1) / L.grid;
  psync::cta_signal_phase(v, L, 0, 1u << peer);
  bool ok = psync::cta_wait_phase(v, L, 0, 1u << peer);
  if (ok) {
    constexpr int U = 4;
    int64_t i = lo + threadIdx.x;
    for (; i + (U - 1) * kThreads < hi; i += U * kThreads) {
      uint4 a[U], b[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        b[u] = peer_in[i + u * kThreads];
        a[u] = in[i + u * kThreads];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float s[O::N];
#pragma unroll
        for (int k = 0; k < O::N; ++k) s[k] = 0.f;
        O::acc(s, a[u]);
        O::acc(s, b[u]);
        out[i + u * kThreads] = O::pack(s, 0.5f);
      }
    }
    for (; i < hi; i += kThreads) {
      float s[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) s[k] = 0.f;
      O::acc(s, in[i]);
      O::acc(s, peer_in[i]);
      out[i] = O::pack(s, 0.5f);
    }
    psync::cta_signal_phase(v, L, 1, 1u << peer);
    ok = psync::cta_wait_phase(v, L, 1, 1u << peer);
  }
  psync::cta_finish_op(v, L);
}

}  // namespace allreduce_bodies
}  // namespace fused
}  // namespace bagua
