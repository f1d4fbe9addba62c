// The device bodies of the fused all-reduce, pair-average and collective kernels, compiled for the host
// (-DBAGUA_HOST_EMULATION) and run with one OS thread per CUDA thread: N ranks x G blocks x
// kThreads threads execute random sequences of these ops over per-rank staging buffers
// and signal pads, every result is checked against the collective's definition, and the
// whole program is meant to be built with -fsanitize=thread, so that a payload access that
// the signalling does not order shows up as a data race.
//
// What it models of a GPU run: the kernel boundary on each rank's stream (a per-rank barrier
// between ops, so ranks drift apart by whole ops), block b of every rank pairing with block
// b of its peers, and the `done` chain that protects staging reuse.
//
//   device_emulation [nranks] [blocks] [ops] [seed] [absent_rank] [deadline_ms] [a2av_mismatch]
//
// With absent_rank >= 0 that rank never runs (a process that died between steps): the others'
// waits must run out after deadline_ms, record what they waited for in the status record, and
// return — the program then exits with code 3 instead of hanging.  With a2av_mismatch = 1 every op is
// an all-to-all with per-pair sizes in which rank 0 announces a longer segment than rank 1 expects:
// rank 1 must report status code 4 and still receive the bytes it asked for (run it with ops = 1).
#include <barrier>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include <cmath>

#include "kernels/fused_allreduce_bodies.cuh"
#include "kernels/fused_allreduce_tma.cuh"
#include "kernels/fused_bytegrad_body.cuh"
#include "kernels/fused_collectives_bodies.cuh"
#include "kernels/fused_gossip_body.cuh"
#include "kernels/fused_nvls_body.cuh"

using namespace bagua;
using namespace bagua::fused;
using namespace bagua::fused::collectives;
using namespace bagua::fused::allreduce_bodies;
using bagua::psync::Launch;

namespace {

enum class Kind {
  AllGather,
  AllGatherInPlace,
  AllGatherSym,
  AllToAll,
  AllToAllInPlace,
  AllToAllSym,
  ReduceScatter,
  ReduceScatterInPlace,
  ReduceScatterSym,
  BroadcastDirect,
  BroadcastTwoPhase,
  Scatter,
  Gather,
  ReduceDirect,
  ReduceTwoPhase,
  Barrier,
  AllReduceOneShot,
  AllReduceTwoShot,
  AllReduceTwoShotInPlace,
  AllReduceSym,
  AllReduceSymTma,
  AllReduceCe,
  AllReduceCeInPlace,
  PairAverage,
  PairAverageSym,
  ByteGrad,
  LpRing,
  AllReduceNvls,
  AllToAllV,
  kCount
};

struct Op {
  Kind kind;
  int64_t vecs;  // per chunk (chunked ops) or per buffer
  int root;
  float scale;
};

float value(uint32_t op, int rank, int64_t i) { return (float)((op * 31u + (uint32_t)rank * 7u + (uint32_t)i) % 1000u); }

struct alignas(16) Vec {
  float f[4];
};

struct Rank {
  std::vector<Vec> staging, in, out, w, l, r;  // w / l / r: the replicas of the low-precision ring
  std::vector<Vec> ce_stage;                   // rank-local staging of the copy-engine all-reduce (never shared)
  std::vector<uint32_t> signals;
  std::unique_ptr<std::barrier<>> bar;  // the rank's stream: all of its threads between ops
  uint64_t errors = 0;
};

struct World {
  int N, G;
  std::vector<Op> ops;
  std::vector<Rank> ranks;
  DeviceStatus status{};
  std::vector<std::unique_ptr<hostemu::BlockContext>> blocks;  // [rank * G + block]
  int absent = -1;
  uint64_t deadline_ns = 60ull * 1000000000ull;
  std::vector<uint64_t> grid_bar_base;  // per op: grid barriers every rank has executed before it, times G
};

// ---- scalar restatement of MinMaxUInt8, independent of the device helpers ----------------
struct Quantiser {
  float scale, lower, upper;
  Quantiser(float mn, float mx) {
    const float denom = (mx - mn) + 1e-7f;
    scale = (float)(255.0 / (double)denom);
    upper = std::rint(mx * scale);
    lower = upper - 255.0f;
  }
  float roundtrip(float x) const {
    float level = std::fmin(std::rint(x * scale), upper);
    const float q = (float)(uint8_t)std::fmin(std::fmax(level - lower, 0.f), 255.f);
    return (q + lower) / scale;
  }
};
Quantiser quantiser_of(const std::vector<float>& v) {
  float mn = v[0], mx = v[0];
  for (float x : v) {
    mn = std::fmin(mn, x);
    mx = std::fmax(mx, x);
  }
  return Quantiser(mn, mx);
}

// Inputs of the low-precision ring for op k on `rank`: x, w, l, r.
float ring_input(uint32_t k, int rank, int which, int64_t i) { return value(k + 17u * (uint32_t)which, rank, i) * 0.125f; }
std::vector<float> ring_difference(uint32_t k, int rank, int64_t n) {
  std::vector<float> d((size_t)n);
  const float third = 1.0f / 3.0f, m53 = -5.0f / 3.0f;
  for (int64_t i = 0; i < n; ++i) {
    float t = std::fmaf(ring_input(k, rank, 2, i), third, ring_input(k, rank, 0, i));
    t = std::fmaf(ring_input(k, rank, 3, i), third, t);
    d[(size_t)i] = std::fmaf(ring_input(k, rank, 1, i), m53, t);
  }
  return d;
}

// All-to-all with per-pair sizes: op k moves a2av_bytes(k, s, d) bytes from s to d, in units of 16, 8,
// 4, 2 or 1 bytes depending on the op, packed back to back on both sides.
constexpr int kA2avMaxUnits = 37;
int64_t a2av_unit(uint32_t k) { return (int64_t)16 >> (k % 5u); }
int64_t a2av_bytes(uint32_t k, int s, int d) {
  return a2av_unit(k) * (int64_t)((k * 7u + (uint32_t)s * 3u + (uint32_t)d * 5u) % (uint32_t)kA2avMaxUnits);
}
bool g_a2av_mismatch = false;  // rank 0 announces one unit more for rank 1 than rank 1 expects
VSegments a2av_segments(uint32_t k, int me, int N) {
  VSegments seg;
  std::memset(&seg, 0, sizeof(seg));
  int64_t so = 0, ro = 0;
  for (int q = 0; q < N; ++q) {
    seg.send_off[q] = so;
    seg.send_bytes[q] = a2av_bytes(k, me, q);
    so += seg.send_bytes[q];
    if (g_a2av_mismatch && me == 0 && q == 1) seg.send_bytes[q] += a2av_unit(k);
    seg.recv_off[q] = ro;
    seg.recv_bytes[q] = a2av_bytes(k, q, me);
    ro += seg.recv_bytes[q];
  }
  return seg;
}
uint8_t input_byte(uint32_t k, int rank, int64_t byte) {
  const float f = value(k, rank, byte / 4);
  uint8_t b[4];
  std::memcpy(b, &f, 4);
  return b[byte % 4];
}

ArenaView view_of(World& w, int rank, uint32_t epoch) {
  ArenaView v;
  std::memset(&v, 0, sizeof(v));
  for (int q = 0; q < w.N; ++q) {
    v.staging[q] = reinterpret_cast<uint8_t*>(w.ranks[q].staging.data());
    v.signals[q] = w.ranks[q].signals.data();
  }
  v.status = &w.status;
  v.staging_bytes = w.ranks[0].staging.size() * sizeof(Vec);
  v.rank = rank;
  v.nranks = w.N;
  v.epoch = epoch;
  v.deadline_ns = w.deadline_ns;
  v.grid_bar_base = w.grid_bar_base[epoch - 1];
  return v;
}

void fill(std::vector<Vec>& buf, uint32_t op, int rank, int64_t vecs) {
  for (int64_t i = 0; i < vecs; ++i)
    for (int l = 0; l < 4; ++l) buf[(size_t)i].f[l] = value(op, rank, 4 * i + l);
}
void poison(std::vector<Vec>& buf) {
  for (auto& x : buf)
    for (int l = 0; l < 4; ++l) x.f[l] = -12345.0f;
}

// Run by one thread of the rank before the op: inputs and poisoned outputs.
void prepare(World& w, int me, uint32_t k) {
  const Op& op = w.ops[k];
  Rank& r = w.ranks[me];
  const int N = w.N;
  poison(r.out);
  switch (op.kind) {
    case Kind::AllGather:
    case Kind::AllGatherSym:
    case Kind::Gather: fill(r.in, k, me, op.vecs); break;
    case Kind::AllGatherInPlace:
      for (int64_t i = 0; i < op.vecs; ++i)
        for (int l = 0; l < 4; ++l) r.out[(size_t)(me * op.vecs + i)].f[l] = value(k, me, 4 * i + l);
      break;
    case Kind::AllToAll:
    case Kind::AllToAllSym:
    case Kind::ReduceScatter:
    case Kind::ReduceScatterInPlace:
    case Kind::ReduceScatterSym:
    case Kind::Scatter: fill(r.in, k, me, op.vecs * N); break;
    case Kind::AllToAllInPlace: fill(r.out, k, me, op.vecs * N); break;
    case Kind::BroadcastDirect:
    case Kind::BroadcastTwoPhase: fill(r.out, k, me, op.vecs); break;  // only the root's content matters
    case Kind::ReduceDirect:
    case Kind::ReduceTwoPhase:
    case Kind::AllReduceOneShot:
    case Kind::AllReduceTwoShot:
    case Kind::AllReduceSym:
    case Kind::AllReduceSymTma:
    case Kind::AllReduceCe:
    case Kind::PairAverage:
    case Kind::PairAverageSym: fill(r.in, k, me, op.vecs); break;
    case Kind::AllReduceCeInPlace:
    case Kind::AllReduceTwoShotInPlace:
    case Kind::AllReduceNvls: fill(r.out, k, me, op.vecs); break;
    case Kind::ByteGrad: fill(r.in, k, me, op.vecs * N); break;
    case Kind::AllToAllV: fill(r.in, k, me, (int64_t)kA2avMaxUnits * N); break;
    case Kind::LpRing:
      for (int64_t i = 0; i < op.vecs; ++i)
        for (int l = 0; l < 4; ++l) {
          r.in[(size_t)i].f[l] = ring_input(k, me, 0, 4 * i + l);
          r.w[(size_t)i].f[l] = ring_input(k, me, 1, 4 * i + l);
          r.l[(size_t)i].f[l] = ring_input(k, me, 2, 4 * i + l);
          r.r[(size_t)i].f[l] = ring_input(k, me, 3, 4 * i + l);
        }
      break;
    default: break;
  }
}

// Run by every thread of the rank: the device body.
void run_body(World& w, int me, int b, uint32_t k) {
  const Op& op = w.ops[k];
  Rank& r = w.ranks[me];
  const ArenaView v = view_of(w, me, k + 1);
  const Launch L{b, w.G};
  const uint4* in = reinterpret_cast<const uint4*>(r.in.data());
  uint4* out = reinterpret_cast<uint4*>(r.out.data());
  PeerPtrs outs;
  ConstPeerPtrs ins;
  for (int q = 0; q < kArenaMaxRanks; ++q) {
    outs.p[q] = q < w.N ? reinterpret_cast<uint4*>(w.ranks[q].out.data()) : nullptr;
    ins.p[q] = q < w.N ? reinterpret_cast<const uint4*>(w.ranks[q].in.data()) : nullptr;
  }
  const int64_t c = op.vecs;
  switch (op.kind) {
    case Kind::AllGather: exchange_body(v, L, in, out, c, 0, 0); break;
    case Kind::AllGatherInPlace: exchange_body(v, L, out + me * c, out, c, 0, 1); break;
    case Kind::AllGatherSym: exchange_sym_body(v, L, in, outs, c, 0, 0); break;
    case Kind::AllToAll: exchange_body(v, L, in, out, c, 1, 0); break;
    case Kind::AllToAllInPlace: exchange_body(v, L, out, out, c, 1, 1); break;
    case Kind::AllToAllSym: exchange_sym_body(v, L, in, outs, c, 1, 0); break;
    case Kind::ReduceScatter: reduce_scatter_body<float>(v, L, in, out, c, op.scale); break;
    case Kind::ReduceScatterInPlace: {
      uint4* io = reinterpret_cast<uint4*>(r.in.data());
      reduce_scatter_body<float>(v, L, io, io + me * c, c, op.scale);
      break;
    }
    case Kind::ReduceScatterSym: reduce_scatter_sym_body<float>(v, L, ins, out, c, op.scale); break;
    case Kind::BroadcastDirect: broadcast_direct_body(v, L, out, c, op.root); break;
    case Kind::BroadcastTwoPhase: broadcast_twophase_body(v, L, out, c, op.root); break;
    case Kind::Scatter: scatter_body(v, L, in, out, c, op.root, 0); break;
    case Kind::Gather: gather_body(v, L, in, out, c, op.root, 0); break;
    case Kind::ReduceDirect: reduce_direct_body<float>(v, L, in, out, c, op.root, op.scale); break;
    case Kind::ReduceTwoPhase:
      reduce_twophase_body<float>(v, L, in, out, c, (c + w.N - 1) / w.N, op.root, op.scale);
      break;
    case Kind::Barrier: barrier_body(v, L); break;
    case Kind::AllReduceOneShot: allreduce_oneshot_body<float>(v, L, in, out, c, c, op.scale); break;
    case Kind::AllReduceTwoShot: allreduce_twoshot_body<float>(v, L, in, out, c, (c + w.N - 1) / w.N, op.scale); break;
    case Kind::AllReduceTwoShotInPlace:
      allreduce_twoshot_body<float>(v, L, out, out, c, (c + w.N - 1) / w.N, op.scale);
      break;
    case Kind::AllReduceSym: {
      SymPtrs p;
      for (int q = 0; q < kArenaMaxRanks; ++q) {
        p.in[q] = ins.p[q];
        p.out[q] = outs.p[q];
      }
      allreduce_sym_body<float>(v, L, p, c, op.scale);
      break;
    }
    case Kind::AllReduceSymTma: {
      // the bulk-copy variant exists for 2, 4 and 8 ranks; other worlds take the load/store body,
      // as the dispatch does
      SymPtrs p;
      for (int q = 0; q < kArenaMaxRanks; ++q) {
        p.in[q] = ins.p[q];
        p.out[q] = outs.p[q];
      }
      constexpr int kSlot = 12;  // the block's dynamic shared memory
      if (w.N == 2)
        allreduce_sym_tma_body<float, 2>(v, L, p, c, op.scale, hostemu::shared_array<unsigned char>(kSlot, TmaCfg<2>::kSmemBytes));
      else if (w.N == 4)
        allreduce_sym_tma_body<float, 4>(v, L, p, c, op.scale, hostemu::shared_array<unsigned char>(kSlot, TmaCfg<4>::kSmemBytes));
      else if (w.N == 8)
        allreduce_sym_tma_body<float, 8>(v, L, p, c, op.scale, hostemu::shared_array<unsigned char>(kSlot, TmaCfg<8>::kSmemBytes));
      else
        allreduce_sym_body<float>(v, L, p, c, op.scale);
      break;
    }
    case Kind::AllReduceCe:
    case Kind::AllReduceCeInPlace: {
      // The copy-engine all-reduce (kernels/fused_allreduce_ce.cu) is a stream of separate launches:
      // one-block sync kernel, N-1 pulls, reduction, N-1 pushes, one-block sync kernel.  Here block 0
      // of the rank plays that stream (a block barrier stands for each launch boundary, thread 0 for
      // the copy engine), the other blocks have nothing to do.  What this checks is the ordering
      // argument: phase 0 before any pull, every push before phase 1, and, in place, that nobody reads
      // a chunk another rank is pushing into.
      if (b != 0) break;
      const Launch one{0, 1};
      const bool in_place = op.kind == Kind::AllReduceCeInPlace;
      const int N = w.N;
      auto lo_of = [&](int q) { return c * q / N; };
      const int64_t my_lo = lo_of(me), my_vecs = lo_of(me + 1) - my_lo, slot = (c + N - 1) / N;
      uint4* stage = reinterpret_cast<uint4*>(r.ce_stage.data());
      psync::cta_signal_phase(v, one, 0, all_peers_mask(v));
      psync::cta_wait_phase(v, one, 0, all_peers_mask(v));
      __syncthreads();
      uint4* own = out + my_lo;
      if (threadIdx.x == 0) {
        for (int i = 1; i < N; ++i) {
          const int q = (me + i) % N;
          const uint4* src = in_place ? outs.p[q] : ins.p[q];
          std::memcpy(stage + (int64_t)q * slot, src + my_lo, (size_t)my_vecs * sizeof(uint4));
        }
        if (!in_place) std::memcpy(own, in + my_lo, (size_t)my_vecs * sizeof(uint4));
      }
      __syncthreads();
      for (int64_t i = threadIdx.x; i < my_vecs; i += kThreads) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        for (int q = 0; q < N; ++q) VecOps<float>::acc(a, q == me ? own[i] : stage[(int64_t)q * slot + i]);
        own[i] = VecOps<float>::pack(a, op.scale);
      }
      __syncthreads();
      if (threadIdx.x == 0)
        for (int i = 1; i < N; ++i) {
          const int q = (me + i) % N;
          std::memcpy(outs.p[q] + my_lo, own, (size_t)my_vecs * sizeof(uint4));
        }
      psync::cta_signal_phase(v, one, 1, all_peers_mask(v));
      psync::cta_wait_phase(v, one, 1, all_peers_mask(v));
      psync::cta_finish_op(v, one);
      break;
    }
    case Kind::PairAverage: pair_average_body<float>(v, L, in, out, c, me ^ 1); break;
    case Kind::PairAverageSym: pair_average_sym_body<float>(v, L, in, ins.p[me ^ 1], out, c, me ^ 1); break;
    case Kind::AllReduceNvls: {
      // in place on the `out` buffers, which stand for memory bound to one multicast object;
      // the multicast address is the one inside rank 0's buffer
      uint4* mc = reinterpret_cast<uint4*>(w.ranks[0].out.data());
      nvls_bodies::allreduce_nvls_body<float>(v, L, mc, mc, c, op.scale);
      break;
    }
    case Kind::AllToAllV: {
      ConstBytePtrs src;
      for (int q = 0; q < kArenaMaxRanks; ++q)
        src.p[q] = q < w.N ? reinterpret_cast<const uint8_t*>(w.ranks[q].in.data()) : nullptr;
      alltoall_v_sym_body(v, L, src, reinterpret_cast<uint8_t*>(r.out.data()), a2av_segments(k, me, w.N));
      break;
    }
    case Kind::ByteGrad: {
      // bucket of N chunks of 4c floats, quantised to one byte each; slots hold a 32-byte header + payload
      const int64_t chunk = 4 * c;
      const size_t slot = (size_t)chunk + 32;
      const size_t scratch_off = ((2 * (size_t)w.N * slot + 255) / 256) * 256;
      // the op's (otherwise unused) root picks the variant: odd = chunks travel back one destination at a time
      bytegrad_bodies::bytegrad_body<float>(v, L, reinterpret_cast<float*>(r.in.data()), chunk, slot, scratch_off,
                                            op.scale, (op.root & 1) != 0);
      break;
    }
    case Kind::LpRing: {
      const int64_t n = 4 * c;
      const size_t slot = (size_t)n + 32;
      const size_t scratch_off = ((3 * slot + 255) / 256) * 256;
      gossip_bodies::lp_ring_body<float>(v, L, reinterpret_cast<float*>(r.in.data()), reinterpret_cast<float*>(r.w.data()),
                                         reinterpret_cast<float*>(r.l.data()), reinterpret_cast<float*>(r.r.data()), n,
                                         slot, scratch_off);
      break;
    }
    default: break;
  }
}

// Run by one thread of the rank after the op (its kernel has finished).
uint64_t verify(World& w, int me, uint32_t k) {
  const Op& op = w.ops[k];
  Rank& r = w.ranks[me];
  const int N = w.N;
  const int64_t c = op.vecs;
  uint64_t bad = 0;
  auto expect = [&](const std::vector<Vec>& buf, int64_t vec, float want_l0, float want_l1, float want_l2, float want_l3) {
    const Vec& x = buf[(size_t)vec];
    if (x.f[0] != want_l0 || x.f[1] != want_l1 || x.f[2] != want_l2 || x.f[3] != want_l3) ++bad;
  };
  auto val4 = [&](int rank, int64_t vec, float* o) {
    for (int l = 0; l < 4; ++l) o[l] = value(k, rank, 4 * vec + l);
  };
  auto sum4 = [&](int64_t vec, float scale, float* o) {
    for (int l = 0; l < 4; ++l) {
      float s = 0.f;
      for (int q = 0; q < N; ++q) s += value(k, q, 4 * vec + l);
      o[l] = s * scale;
    }
  };
  float e[4];
  switch (op.kind) {
    case Kind::AllGather:
    case Kind::AllGatherInPlace:
    case Kind::AllGatherSym:
      for (int q = 0; q < N; ++q)
        for (int64_t i = 0; i < c; ++i) {
          val4(q, i, e);
          expect(r.out, q * c + i, e[0], e[1], e[2], e[3]);
        }
      break;
    case Kind::AllToAll:
    case Kind::AllToAllInPlace:
    case Kind::AllToAllSym:
      for (int q = 0; q < N; ++q)
        for (int64_t i = 0; i < c; ++i) {
          val4(q, me * c + i, e);
          expect(r.out, q * c + i, e[0], e[1], e[2], e[3]);
        }
      break;
    case Kind::ReduceScatter:
    case Kind::ReduceScatterSym:
      for (int64_t i = 0; i < c; ++i) {
        sum4(me * c + i, op.scale, e);
        expect(r.out, i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::ReduceScatterInPlace:
      for (int64_t i = 0; i < c; ++i) {
        sum4(me * c + i, op.scale, e);
        expect(r.in, me * c + i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::BroadcastDirect:
    case Kind::BroadcastTwoPhase:
      for (int64_t i = 0; i < c; ++i) {
        val4(op.root, i, e);
        expect(r.out, i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::Scatter:
      for (int64_t i = 0; i < c; ++i) {
        val4(op.root, me * c + i, e);
        expect(r.out, i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::Gather:
      if (me == op.root)
        for (int q = 0; q < N; ++q)
          for (int64_t i = 0; i < c; ++i) {
            val4(q, i, e);
            expect(r.out, q * c + i, e[0], e[1], e[2], e[3]);
          }
      else
        for (int64_t i = 0; i < c * N; ++i) expect(r.out, i, -12345.0f, -12345.0f, -12345.0f, -12345.0f);
      break;
    case Kind::ReduceDirect:
    case Kind::ReduceTwoPhase:
      for (int64_t i = 0; i < c; ++i) {
        if (me == op.root) {
          sum4(i, op.scale, e);
          expect(r.out, i, e[0], e[1], e[2], e[3]);
        } else {
          expect(r.out, i, -12345.0f, -12345.0f, -12345.0f, -12345.0f);
        }
      }
      break;
    case Kind::AllReduceOneShot:
    case Kind::AllReduceTwoShot:
    case Kind::AllReduceTwoShotInPlace:
    case Kind::AllReduceSym:
    case Kind::AllReduceSymTma:
    case Kind::AllReduceCe:
    case Kind::AllReduceCeInPlace:
    case Kind::AllReduceNvls:
      for (int64_t i = 0; i < c; ++i) {
        sum4(i, op.scale, e);
        expect(r.out, i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::PairAverage:
    case Kind::PairAverageSym:
      for (int64_t i = 0; i < c; ++i) {
        for (int l = 0; l < 4; ++l) e[l] = (value(k, me, 4 * i + l) + value(k, me ^ 1, 4 * i + l)) * 0.5f;
        expect(r.out, i, e[0], e[1], e[2], e[3]);
      }
      break;
    case Kind::ByteGrad: {
      // every rank's chunk ch is quantised with its own grid, the owner sums the N dequantised
      // contributions in rank order, scales, quantises the result once more; all ranks end up with that
      const int64_t chunk = 4 * c;
      const float* got = reinterpret_cast<const float*>(r.in.data());
      for (int ch = 0; ch < N; ++ch) {
        std::vector<float> reduced((size_t)chunk, 0.f);
        for (int q = 0; q < N; ++q) {
          std::vector<float> contrib((size_t)chunk);
          for (int64_t i = 0; i < chunk; ++i) contrib[(size_t)i] = value(k, q, ch * chunk + i);
          const Quantiser g = quantiser_of(contrib);
          for (int64_t i = 0; i < chunk; ++i) reduced[(size_t)i] += g.roundtrip(contrib[(size_t)i]);
        }
        for (auto& x : reduced) x *= op.scale;
        const Quantiser g2 = quantiser_of(reduced);
        for (int64_t i = 0; i < chunk; ++i)
          if (got[ch * chunk + i] != g2.roundtrip(reduced[(size_t)i])) ++bad;
      }
      break;
    }
    case Kind::AllToAllV: {
      const VSegments seg = a2av_segments(k, me, N);
      const uint8_t* got = reinterpret_cast<const uint8_t*>(r.out.data());
      int64_t end = 0;
      for (int q = 0; q < N; ++q) {
        const VSegments theirs = a2av_segments(k, q, N);
        for (int64_t j = 0; j < seg.recv_bytes[q]; ++j)
          if (got[seg.recv_off[q] + j] != input_byte(k, q, theirs.send_off[me] + j)) ++bad;
        end = seg.recv_off[q] + seg.recv_bytes[q];
      }
      // nothing behind the last segment may have been touched
      const float poison_value = -12345.0f;
      uint8_t pb[4];
      std::memcpy(pb, &poison_value, 4);
      for (int64_t j = end; j < (int64_t)(r.out.size() * sizeof(Vec)); ++j)
        if (got[j] != pb[j % 4]) {
          ++bad;
          break;
        }
      break;
    }
    case Kind::LpRing: {
      const int64_t n = 4 * c;
      const int left = (me + N - 1) % N, right = (me + 1) % N;
      const std::vector<float> d_me = ring_difference(k, me, n), d_l = ring_difference(k, left, n),
                               d_r = ring_difference(k, right, n);
      const Quantiser g_me = quantiser_of(d_me), g_l = quantiser_of(d_l), g_r = quantiser_of(d_r);
      const float* x = reinterpret_cast<const float*>(r.in.data());
      const float* wv = reinterpret_cast<const float*>(r.w.data());
      const float* lv = reinterpret_cast<const float*>(r.l.data());
      const float* rv = reinterpret_cast<const float*>(r.r.data());
      for (int64_t i = 0; i < n; ++i) {
        const float nw = g_me.roundtrip(d_me[(size_t)i]) + ring_input(k, me, 1, i);
        if (x[i] != nw || wv[i] != nw) ++bad;
        if (lv[i] != ring_input(k, me, 2, i) + g_l.roundtrip(d_l[(size_t)i])) ++bad;
        if (rv[i] != ring_input(k, me, 3, i) + g_r.roundtrip(d_r[(size_t)i])) ++bad;
      }
      break;
    }
    default: break;
  }

  // Stray stores: `out` was poisoned before the op, so everything past the op's output must
  // still be poison; and an op that is not in place must leave its input as it was.
  int64_t out_extent = 0, in_extent = 0;
  switch (op.kind) {
    case Kind::AllGather:
    case Kind::AllGatherSym: out_extent = c * N, in_extent = c; break;
    case Kind::AllGatherInPlace:
    case Kind::AllToAllInPlace: out_extent = c * N; break;
    case Kind::AllToAll:
    case Kind::AllToAllSym: out_extent = c * N, in_extent = c * N; break;
    case Kind::ReduceScatter:
    case Kind::ReduceScatterSym: out_extent = c, in_extent = c * N; break;
    case Kind::BroadcastDirect:
    case Kind::BroadcastTwoPhase: out_extent = c; break;
    case Kind::Scatter: out_extent = c, in_extent = me == op.root ? c * N : 0; break;
    case Kind::Gather: out_extent = me == op.root ? c * N : 0, in_extent = c; break;
    case Kind::ReduceDirect:
    case Kind::ReduceTwoPhase: out_extent = me == op.root ? c : 0, in_extent = c; break;
    case Kind::AllReduceOneShot:
    case Kind::AllReduceTwoShot:
    case Kind::AllReduceSym:
    case Kind::AllReduceSymTma:
    case Kind::AllReduceCe:
    case Kind::PairAverage:
    case Kind::PairAverageSym: out_extent = c, in_extent = c; break;
    case Kind::AllReduceCeInPlace:
    case Kind::AllReduceTwoShotInPlace:
    case Kind::AllReduceNvls: out_extent = c; break;
    case Kind::AllToAllV: out_extent = (int64_t)r.out.size(), in_extent = (int64_t)kA2avMaxUnits * N; break;  // bytes checked above
    default: break;  // ReduceScatterInPlace, ByteGrad, LpRing, Barrier: `out` is not touched
  }
  for (int64_t i = out_extent; i < (int64_t)r.out.size(); ++i) expect(r.out, i, -12345.0f, -12345.0f, -12345.0f, -12345.0f);
  for (int64_t i = 0; i < in_extent; ++i) {
    val4(me, i, e);
    expect(r.in, i, e[0], e[1], e[2], e[3]);
  }
  return bad;
}

void cuda_thread(World& w, int me, int b, int t) {
  hostemu::bind_thread(w.blocks[(size_t)(me * w.G + b)].get(), (unsigned)t, (unsigned)b, (unsigned)w.G);
  Rank& r = w.ranks[me];
  const bool lead = b == 0 && t == 0;
  if (me == w.absent) return;
  for (uint32_t k = 0; k < w.ops.size(); ++k) {
    if (lead) prepare(w, me, k);
    r.bar->arrive_and_wait();  // inputs ready: the kernel starts on this rank
    run_body(w, me, b, k);
    r.bar->arrive_and_wait();  // kernel boundary: every block of this rank has finished
    if (lead && w.absent < 0) r.errors += verify(w, me, k);
  }
}

}  // namespace

int main(int argc, char** argv) {
  World w;
  w.N = argc > 1 ? std::atoi(argv[1]) : 4;
  w.G = argc > 2 ? std::atoi(argv[2]) : 2;
  const int n_ops = argc > 3 ? std::atoi(argv[3]) : 64;
  const uint32_t seed = argc > 4 ? (uint32_t)std::atoi(argv[4]) : 1;
  w.absent = argc > 5 ? std::atoi(argv[5]) : -1;
  if (argc > 6) w.deadline_ns = (uint64_t)std::atoll(argv[6]) * 1000000ull;
  g_a2av_mismatch = argc > 7 && std::atoi(argv[7]) != 0;
  if (w.N < 2 || w.N > kArenaMaxRanks || w.G < 1 || w.G > 8 || n_ops < 1 || w.absent >= w.N) {
    std::fprintf(stderr, "usage: device_emulation [nranks 2..8] [blocks 1..8] [ops] [seed] [absent_rank] [deadline_ms]\n");
    return 2;
  }
  std::mt19937 rng(seed);
  int64_t max_vecs = 0;
  for (int k = 0; k < n_ops; ++k) {
    Op op;
    op.kind = (Kind)(rng() % (uint32_t)Kind::kCount);
    if ((op.kind == Kind::PairAverage || op.kind == Kind::PairAverageSym) && w.N % 2) op.kind = Kind::Barrier;  // pairs need an even world
    op.vecs = 1 + (int64_t)(rng() % 40);
    if (op.kind == Kind::ByteGrad || op.kind == Kind::LpRing) op.vecs = 4 * (1 + (int64_t)(rng() % 10));  // 16-element groups
    if (op.kind == Kind::AllReduceSymTma || op.kind == Kind::AllReduceCe || op.kind == Kind::AllReduceCeInPlace) op.vecs = 1 + (int64_t)(rng() % 400);  // many tiles: the stage ring wraps
    if (g_a2av_mismatch) op.kind = Kind::AllToAllV;
    if (op.kind == Kind::AllToAllV) op.vecs = kA2avMaxUnits;  // sizes the buffers; the op's own sizes come from a2av_bytes
    op.root = (int)(rng() % (uint32_t)w.N);
    op.scale = (rng() & 1) ? 1.0f : 0.5f;
    max_vecs = std::max(max_vecs, op.vecs);
    w.grid_bar_base.push_back(w.grid_bar_base.empty() ? 0 : w.grid_bar_base.back());
    if (!w.ops.empty()) {
      const Kind prev = w.ops.back().kind;
      w.grid_bar_base.back() += (uint64_t)w.G * (prev == Kind::ByteGrad ? 2u : prev == Kind::LpRing ? 1u : 0u);
    }
    w.ops.push_back(op);
  }
  const size_t buf_vecs = (size_t)max_vecs * (size_t)w.N;
  w.ranks.resize((size_t)w.N);
  for (auto& r : w.ranks) {
    r.staging.assign(buf_vecs * 2 + 64 + (size_t)(w.N + 1) * (size_t)w.G, Vec{});  // slots, mirror areas, min/max scratch
    r.in.assign(buf_vecs, Vec{});
    r.out.assign(buf_vecs, Vec{});
    r.w.assign(buf_vecs, Vec{});
    r.l.assign(buf_vecs, Vec{});
    r.r.assign(buf_vecs, Vec{});
    r.ce_stage.assign(buf_vecs + (size_t)w.N, Vec{});
    r.signals.assign((size_t)kSigWords, 0u);
    r.bar = std::make_unique<std::barrier<>>(w.G * kThreads);
  }
  nvls_bodies::g_host_multicast.nranks = w.N;
  for (int q = 0; q < w.N; ++q) nvls_bodies::g_host_multicast.base[q] = reinterpret_cast<char*>(w.ranks[(size_t)q].out.data());
  for (int i = 0; i < w.N * w.G; ++i) w.blocks.push_back(std::make_unique<hostemu::BlockContext>(kThreads));

  std::vector<std::thread> threads;
  for (int r = 0; r < w.N; ++r)
    for (int b = 0; b < w.G; ++b)
      for (int t = 0; t < kThreads; ++t) threads.emplace_back(cuda_thread, std::ref(w), r, b, t);
  for (auto& t : threads) t.join();

  uint64_t errors = 0;
  for (auto& r : w.ranks) errors += r.errors;
  if (w.absent >= 0) {
    std::printf("device emulation: rank %d absent, every other rank returned; wait status code %u (phase %u, peer %u)\n",
                w.absent, w.status.code, w.status.phase, w.status.peer);
    return w.status.code != 0 ? 3 : 1;
  }
  const int failures = (errors != 0) + (w.status.code != 0);
  std::printf("device emulation: %d ranks x %d blocks x %d threads, %d ops, %llu wrong vectors, wait status %u, %d failures\n",
              w.N, w.G, kThreads, n_ops, (unsigned long long)errors, w.status.code, failures);
  return failures ? 1 : 0;
}
