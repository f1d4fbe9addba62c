// Device bodies of the peer-memory collective kernels (see fused_collectives.cu for the
// algorithms).  Kept in a header so that the same source is compiled twice: by nvcc into the
// sm_100a kernels, and by the host compiler (-DBAGUA_HOST_EMULATION, host_emulation.h) into
// a thread-per-CUDA-thread program that runs every body under ThreadSanitizer
// (tests/cpp/device_emulation.cc).
#pragma once

#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {
namespace collectives {

using psync::Launch;

struct PeerPtrs {
  uint4* p[kArenaMaxRanks];
};

// Vector range of block b inside a chunk of `len` vectors that starts at vector c0.
__device__ __forceinline__ void block_slice(const Launch& L, int64_t c0, int64_t len, int64_t& lo, int64_t& hi) {
  lo = c0 + len * L.block / L.grid;
  hi = c0 + len * (L.block + 1) / L.grid;
}

// ---------------------------------------------------------------------------------
// exchange: out[r] = chunk that rank r holds for me.  src_stride = 0: every peer gets
// in[0..cvec) (all-gather); src_stride = 1: peer q gets in[q*cvec..) (all-to-all).
// ---------------------------------------------------------------------------------
// `in` and `out` may overlap (in-place forms), so neither is declared restrict.
__device__ __forceinline__ void exchange_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                              int64_t cvec, int src_stride, int skip_local) {
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      uint4* dst = reinterpret_cast<uint4*>(v.staging[q]) + (int64_t)me * cvec;
      copy_vecs(dst, in + (int64_t)src_stride * q * cvec, lo, hi);
    }
    if (!skip_local) copy_vecs(out + (int64_t)me * cvec, in + (int64_t)src_stride * me * cvec, lo, hi);
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
    for (int i = 1; i < N; ++i) {
      const int r = (me + i) % N;
      copy_vecs(out + (int64_t)r * cvec, mine + (int64_t)r * cvec, lo, hi);
    }
  }
  psync::cta_finish_op(v, L);
}

// Output in the symmetric heap: store straight into every rank's output.  First signal:
// the peer has started, so its output may be overwritten; second signal: all stores into
// my output have landed.
__device__ __forceinline__ void exchange_sym_body(const ArenaView& v, const Launch& L, const uint4* in,
                                                  const PeerPtrs& out, int64_t cvec, int src_stride,
                                                  int skip_local) {
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  bool ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  if (ok) {
    for (int i = skip_local ? 1 : 0; i < N; ++i) {
      const int q = (me + i) % N;
      copy_vecs(out.p[q] + (int64_t)me * cvec, in + (int64_t)src_stride * q * cvec, lo, hi);
    }
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// reduce-scatter: out[0..cvec) = scale * sum_r in_r[me*cvec ..)
// ---------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void reduce_scatter_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                                    int64_t cvec, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      uint4* dst = reinterpret_cast<uint4*>(v.staging[q]) + (int64_t)me * cvec;
      copy_vecs(dst, in + (int64_t)q * cvec, lo, hi);
    }
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
    const uint4* own = in + (int64_t)me * cvec;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) {
        const uint4 x = (r == me) ? own[i] : mine[(int64_t)r * cvec + i];
        O::acc(a, x);
      }
      out[i] = O::pack(a, scale);  // may alias own[i] (in-place form): read above, same thread
    }
  }
  psync::cta_finish_op(v, L);
}

struct ConstPeerPtrs {
  const uint4* p[kArenaMaxRanks];
};

// Input in the symmetric heap: load chunk `me` of every rank's input directly.  The second
// signal tells the peers that their input is no longer being read.
template <typename T>
__device__ __forceinline__ void reduce_scatter_sym_body(const ArenaView& v, const Launch& L, const ConstPeerPtrs& in,
                                                        uint4* out, int64_t cvec, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  bool ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  if (ok) {
    const int64_t base = (int64_t)me * cvec;
    constexpr int U = 2;
    int64_t i = lo + threadIdx.x;
    for (; i + (U - 1) * kThreads < hi; i += U * kThreads) {
      uint4 x[U][kArenaMaxRanks];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < kArenaMaxRanks; ++r)
          if (r < N) x[u][r] = in.p[r][base + i + u * kThreads];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float a[O::N];
#pragma unroll
        for (int k = 0; k < O::N; ++k) a[k] = 0.f;
#pragma unroll
        for (int r = 0; r < kArenaMaxRanks; ++r)
          if (r < N) O::acc(a, x[u][r]);
        out[i + u * kThreads] = O::pack(a, scale);
      }
    }
    for (; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) O::acc(a, in.p[r][base + i]);
      out[i] = O::pack(a, scale);
    }
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// broadcast (in place on `buf`)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void broadcast_direct_body(const ArenaView& v, const Launch& L, uint4* buf, int64_t nvec,
                                                      int root) {
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, nvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    if (me == root) {
      for (int i = 1; i < N; ++i) {
        const int q = (me + i) % N;
        copy_vecs(reinterpret_cast<uint4*>(v.staging[q]), buf, lo, hi);
      }
      psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    } else {
      ok = psync::cta_wait_phase(v, L, 0, 1u << root);
      if (ok) copy_vecs(buf, reinterpret_cast<const uint4*>(v.staging[me]), lo, hi);
    }
  }
  psync::cta_finish_op(v, L);
}

__device__ __forceinline__ void broadcast_twophase_body(const ArenaView& v, const Launch& L, uint4* buf, int64_t nvec,
                                                        int root) {
  const int me = v.rank, N = v.nranks;
  auto chunk_lo = [&](int c) { return nvec * c / N; };
  auto slice = [&](int c, int64_t& lo, int64_t& hi) {
    const int64_t c0 = chunk_lo(c);
    block_slice(L, c0, chunk_lo(c + 1) - c0, lo, hi);
  };
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    if (me == root) {
      // chunk q goes to q; the root's own chunk goes to everyone (staging mirrors buf's indexing)
      for (int i = 1; i < N; ++i) {
        const int q = (me + i) % N;
        uint4* dst = reinterpret_cast<uint4*>(v.staging[q]);
        int64_t lo, hi;
        slice(q, lo, hi);
        copy_vecs(dst, buf, lo, hi);
        slice(root, lo, hi);
        copy_vecs(dst, buf, lo, hi);
      }
      psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    } else {
      const uint32_t others = all_peers_mask(v) & ~(1u << root);
      ok = psync::cta_wait_phase(v, L, 0, 1u << root);
      if (ok) {
        // forward the chunk I own to everyone but the root
        const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
        int64_t lo, hi;
        slice(me, lo, hi);
        for (int i = 1; i < N; ++i) {
          const int q = (me + i) % N;
          if (q == root) continue;
          copy_vecs(reinterpret_cast<uint4*>(v.staging[q]), mine, lo, hi);
        }
        psync::cta_signal_phase(v, L, 1, others);
        ok = psync::cta_wait_phase(v, L, 1, others);
      }
      if (ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
        for (int c = 0; c < N; ++c) {
          int64_t lo, hi;
          slice(c, lo, hi);
          copy_vecs(buf, mine, lo, hi);
        }
      }
    }
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// scatter / gather: one rank's N chunks to / from the N ranks
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void scatter_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                             int64_t cvec, int root, int skip_local) {
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    if (me == root) {
      for (int i = 1; i < N; ++i) {
        const int q = (me + i) % N;
        copy_vecs(reinterpret_cast<uint4*>(v.staging[q]), in + (int64_t)q * cvec, lo, hi);
      }
      if (!skip_local) copy_vecs(out, in + (int64_t)me * cvec, lo, hi);
      psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    } else {
      ok = psync::cta_wait_phase(v, L, 0, 1u << root);
      if (ok) copy_vecs(out, reinterpret_cast<const uint4*>(v.staging[me]), lo, hi);
    }
  }
  psync::cta_finish_op(v, L);
}

__device__ __forceinline__ void gather_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                            int64_t cvec, int root, int skip_local) {
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, cvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    if (me != root) {
      copy_vecs(reinterpret_cast<uint4*>(v.staging[root]) + (int64_t)me * cvec, in, lo, hi);
      psync::cta_signal_phase(v, L, 0, 1u << root);
    } else {
      if (!skip_local) copy_vecs(out + (int64_t)me * cvec, in, lo, hi);
      ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
      if (ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
        for (int i = 1; i < N; ++i) {
          const int r = (me + i) % N;
          copy_vecs(out + (int64_t)r * cvec, mine + (int64_t)r * cvec, lo, hi);
        }
      }
    }
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// reduce to one rank: out (on root) = scale * sum_r in_r; other ranks' `out` is untouched
// ---------------------------------------------------------------------------------
// Small buffers: everyone stores its whole input into the root's staging.
template <typename T>
__device__ __forceinline__ void reduce_direct_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                                   int64_t nvec, int root, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  int64_t lo, hi;
  block_slice(L, 0, nvec, lo, hi);
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    if (me != root) {
      copy_vecs(reinterpret_cast<uint4*>(v.staging[root]) + (int64_t)me * nvec, in, lo, hi);
      psync::cta_signal_phase(v, L, 0, 1u << root);
    } else {
      ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
      if (ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
        for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
          float a[O::N];
#pragma unroll
          for (int k = 0; k < O::N; ++k) a[k] = 0.f;
          for (int r = 0; r < N; ++r) {
            const uint4 x = (r == me) ? in[i] : mine[(int64_t)r * nvec + i];
            O::acc(a, x);
          }
          out[i] = O::pack(a, scale);
        }
      }
    }
  }
  psync::cta_finish_op(v, L);
}

// Large buffers: reduce-scatter among all ranks, then every rank hands its reduced chunk to
// the root, which receives 2(N-1)/N·S instead of (N-1)·S.  Staging layout as in the two-shot
// all-reduce: N slots of max_chunk vectors, then an area that mirrors the buffer's indexing.
template <typename T>
__device__ __forceinline__ void reduce_twophase_body(const ArenaView& v, const Launch& L, const uint4* in, uint4* out,
                                                     int64_t nvec, int64_t max_chunk_vecs, int root, float scale) {
  using O = VecOps<T>;
  const int me = v.rank, N = v.nranks;
  auto chunk_lo = [&](int c) { return nvec * c / N; };
  auto slice = [&](int c, int64_t& lo, int64_t& hi) {
    const int64_t c0 = chunk_lo(c);
    block_slice(L, c0, chunk_lo(c + 1) - c0, lo, hi);
  };
  const int64_t ag_base = (int64_t)N * max_chunk_vecs;
  bool ok = psync::cta_wait_prev_done(v, L);
  if (ok) {
    for (int i = 1; i < N; ++i) {
      const int q = (me + i) % N;
      int64_t lo, hi;
      slice(q, lo, hi);
      uint4* dst = reinterpret_cast<uint4*>(v.staging[q]) + (int64_t)me * max_chunk_vecs - chunk_lo(q);
      copy_vecs(dst, in, lo, hi);
    }
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    int64_t lo, hi;
    slice(me, lo, hi);
    const int64_t c0 = chunk_lo(me);
    const uint4* mine = reinterpret_cast<const uint4*>(v.staging[me]);
    uint4* dst = (me == root) ? out : reinterpret_cast<uint4*>(v.staging[root]) + ag_base;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float a[O::N];
#pragma unroll
      for (int k = 0; k < O::N; ++k) a[k] = 0.f;
      for (int r = 0; r < N; ++r) {
        const uint4 x = (r == me) ? in[i] : mine[(int64_t)r * max_chunk_vecs + (i - c0)];
        O::acc(a, x);
      }
      dst[i] = O::pack(a, scale);
    }
    if (me != root) {
      psync::cta_signal_phase(v, L, 1, 1u << root);
    } else {
      ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
      if (ok) {
        const uint4* ag = mine + ag_base;
        for (int k = 1; k < N; ++k) {
          const int q = (me + k) % N;
          slice(q, lo, hi);
          copy_vecs(out, ag, lo, hi);
        }
      }
    }
  }
  psync::cta_finish_op(v, L);
}

// ---------------------------------------------------------------------------------
// all-to-all with per-pair sizes, send buffer in the symmetric heap (pull)
// ---------------------------------------------------------------------------------
// Byte offsets and lengths of the segments one rank sends to / receives from each rank.
struct VSegments {
  int64_t send_off[kArenaMaxRanks], send_bytes[kArenaMaxRanks];
  int64_t recv_off[kArenaMaxRanks], recv_bytes[kArenaMaxRanks];
};
struct ConstBytePtrs {
  const uint8_t* p[kArenaMaxRanks];
};

// Block b's share of a copy of `bytes` bytes, in the widest unit (16, 8, 4, 2 or 1 bytes) that
// divides both addresses and the length: segments of whole 16-byte rows move as vectors, anything
// else still arrives, only slower.
template <typename U>
__device__ __forceinline__ void copy_units(uint8_t* dst, const uint8_t* src, int64_t lo, int64_t hi) {
  U* d = reinterpret_cast<U*>(dst);
  const U* s = reinterpret_cast<const U*>(src);
  for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) d[i] = s[i];
}
__device__ __forceinline__ void copy_bytes_slice(const Launch& L, uint8_t* dst, const uint8_t* src, int64_t bytes) {
  const uint64_t mix = (uint64_t)(uintptr_t)dst | (uint64_t)(uintptr_t)src | (uint64_t)bytes;
  const int shift = (mix & 15) == 0 ? 4 : (mix & 7) == 0 ? 3 : (mix & 3) == 0 ? 2 : (mix & 1) == 0 ? 1 : 0;
  int64_t lo, hi;
  block_slice(L, 0, bytes >> shift, lo, hi);
  switch (shift) {
    case 4: copy_vecs(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src), lo, hi); break;
    case 3: copy_units<uint64_t>(dst, src, lo, hi); break;
    case 2: copy_units<uint32_t>(dst, src, lo, hi); break;
    case 1: copy_units<uint16_t>(dst, src, lo, hi); break;
    default: copy_units<uint8_t>(dst, src, lo, hi); break;
  }
}

// Every rank tells every peer where that peer's segment starts in its send buffer and how long
// it is (two words in the peer's staging; only the receiver knows where the data goes), then
// pulls its own segments straight out of the peers' send buffers.  First signal: "my table
// entry for you is written and my send buffer is ready"; second signal: "I have finished
// reading your send buffer".  A receiver that expected another length than the sender
// announced moves the shorter of the two and reports status code 4.
__device__ __forceinline__ void alltoall_v_sym_body(const ArenaView& v, const Launch& L, const ConstBytePtrs& in,
                                                    uint8_t* out, const VSegments& seg) {
  const int me = v.rank, N = v.nranks, t = threadIdx.x;
  bool ok = psync::cta_wait_prev_done(v, L);  // the table lives in staging
  if (ok) {
    if (t < N && t != me) {
      int64_t* entry = reinterpret_cast<int64_t*>(v.staging[t]) + 2 * me;
      same_value_store(entry, seg.send_off[t]);  // every block writes the same two words
      same_value_store(entry + 1, seg.send_bytes[t]);
    }
    psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  }
  if (ok) {
    const int64_t* table = reinterpret_cast<const int64_t*>(v.staging[me]);
    for (int i = 0; i < N; ++i) {
      const int r = (me + i) % N;
      const int64_t off = r == me ? seg.send_off[me] : same_value_load(table + 2 * r);
      int64_t bytes = r == me ? seg.send_bytes[me] : same_value_load(table + 2 * r + 1);
      if (bytes != seg.recv_bytes[r]) {
        if (t == 0) psync::record_timeout(v, 4, 0, (uint32_t)r, (uint32_t)bytes, (uint32_t)L.block);
        bytes = bytes < seg.recv_bytes[r] ? bytes : seg.recv_bytes[r];
      }
      copy_bytes_slice(L, out + seg.recv_off[r], in.p[r] + off, bytes);
    }
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

__device__ __forceinline__ void barrier_body(const ArenaView& v, const Launch& L) {
  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  psync::cta_wait_phase(v, L, 0, all_peers_mask(v));
  psync::cta_finish_op(v, L);
}

}  // namespace collectives
}  // namespace fused
}  // namespace bagua
