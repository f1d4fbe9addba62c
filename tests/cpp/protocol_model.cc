// Host-thread model of the cross-GPU signalling protocol used by the fused kernels.
//
// A test program (tests/test_cpu_protocol_model.py builds it with g++): the kernels' memory
// ordering cannot be checked by a device-side tool here, so the protocol (epoch-valued phase
// words, the `done` chain that guards staging reuse, block-to-block pairing) is restated
// here with std::thread + std::atomic and the same acquire/release structure and the same
// index arithmetic as the kernels, and run under randomised and adversarial schedules:
//   * every (rank, block) pair is a thread; payload words are relaxed atomics (the GPU's
//     weak accesses), signal words use release stores / acquire loads;
//   * a run is a sequence of ops.  With `mix = false` it alternates the one-shot and the
//     two-shot all-reduce, so consecutive ops reuse the same staging addresses for different
//     purposes; with `mix = true` it draws from every kernel of the communicator: the two
//     all-reduces, all-gather, all-to-all and reduce-scatter through staging, all-gather into
//     and reduce-scatter out of peer-visible ("symmetric") buffers, both broadcasts and the
//     barrier;
//   * inputs depend on (op, rank, index): any premature overwrite or stale read shows up
//     as a wrong value; every wait is bounded and counted when it runs out.
// With `use_done_chain = false` the model drops the wait on the peers' `done` words; an
// adversarial delay then corrupts results, which shows that the chain is what makes the
// reuse safe.
#include <atomic>
#include <chrono>
#include <random>
#include <thread>

#include "protocol_model.h"

namespace bagua {

namespace {

enum class Kind {
  TwoShot,
  OneShot,
  AllGather,
  AllToAll,
  ReduceScatter,
  AllGatherSym,
  ReduceScatterSym,
  BroadcastDirect,
  BroadcastTwoPhase,
  Barrier,
  Scatter,
  Gather,
  ReduceDirect,
  ReduceTwoPhase,
  kCount
};

struct RankMem {
  std::vector<std::atomic<uint32_t>> staging;
  std::vector<std::atomic<uint32_t>> sym;     // peer-visible user buffer (symmetric heap)
  std::vector<std::atomic<uint32_t>> done;    // [nranks]
  std::vector<std::atomic<uint32_t>> phase;   // [2][nranks][blocks]
  std::atomic<uint32_t> counter{0};
  RankMem(size_t stage_words, size_t sym_words, int nranks, int blocks)
      : staging(stage_words), sym(sym_words), done((size_t)nranks), phase((size_t)2 * nranks * blocks) {
    for (auto& a : staging) a.store(0xdeadbeefu);
    for (auto& a : sym) a.store(0xfeedf00du);
    for (auto& a : done) a.store(0);
    for (auto& a : phase) a.store(0);
  }
};

struct Model {
  int N, G;
  bool use_done;
  int slow_rank;
  std::vector<std::unique_ptr<RankMem>> mem;
  std::atomic<uint64_t> errors{0}, timeouts{0};

  std::atomic<uint32_t>& phase(int rank, int ph, int src, int block) {
    return mem[rank]->phase[((size_t)ph * N + src) * G + block];
  }
  bool wait(std::atomic<uint32_t>& w, uint32_t want) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(20);
    for (uint64_t spins = 0;; ++spins) {
      if ((int32_t)(w.load(std::memory_order_acquire) - want) >= 0) return true;
      if ((spins & 255) == 0) {
        if (std::chrono::steady_clock::now() > deadline) {
          timeouts++;
          return false;
        }
        std::this_thread::yield();
      }
    }
  }
  static uint32_t input(uint32_t op, int rank, int64_t i) { return op * 1000003u + (uint32_t)rank * 7919u + (uint32_t)i; }
};

struct OpDesc {
  Kind kind;
  int64_t nvec;  // whole-buffer ops: words per rank; chunked ops: words per chunk
  int root;
};

// One block of one rank running the whole op sequence.
struct Block {
  Model& m;
  const int me, b, N, G;
  RankMem& mine;
  std::mt19937 rng;
  uint32_t k = 0, epoch = 0;
  uint64_t bad = 0;

  Block(Model& model, int rank, int block, uint32_t seed)
      : m(model), me(rank), b(block), N(model.N), G(model.G), mine(*model.mem[rank]), rng(seed) {}

  void jitter(int max_us) {
    if (max_us > 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % (uint32_t)max_us));
  }
  uint32_t in(int64_t i) const { return Model::input(k, me, i); }
  uint32_t all_peers() const { return ((1u << N) - 1u) & ~(1u << me); }
  void signal(int ph, uint32_t mask) {
    for (int q = 0; q < N; ++q)
      if ((mask >> q) & 1u) m.phase(q, ph, me, b).store(epoch, std::memory_order_release);
  }
  bool wait_phase(int ph, uint32_t mask) {
    for (int q = 0; q < N; ++q)
      if (((mask >> q) & 1u) && !m.wait(m.phase(me, ph, q, b), epoch)) return false;
    return true;
  }
  bool wait_prev_done() {
    if (!m.use_done) return true;
    for (int q = 0; q < N; ++q)
      if (q != me && !m.wait(mine.done[q], epoch - 1)) return false;
    return true;
  }
  void slice(int64_t c0, int64_t len, int64_t& lo, int64_t& hi) const {
    lo = c0 + len * b / G;
    hi = c0 + len * (b + 1) / G;
  }
  static void put(std::atomic<uint32_t>& w, uint32_t v) { w.store(v, std::memory_order_relaxed); }
  static uint32_t get(const std::atomic<uint32_t>& w) { return w.load(std::memory_order_relaxed); }

  bool oneshot(int64_t nvec) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, nvec, lo, hi);
    for (int s = 1; s < N; ++s) {
      const int q = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)me * nvec + i], in(i));
    }
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int64_t i = lo; i < hi; ++i) {
      uint32_t sum = 0, expect = 0;
      for (int r = 0; r < N; ++r) {
        sum += (r == me) ? in(i) : get(mine.staging[(size_t)r * nvec + i]);
        expect += Model::input(k, r, i);
      }
      if (sum != expect) ++bad;
    }
    return true;
  }

  bool twoshot(int64_t nvec) {
    if (!wait_prev_done()) return false;
    const int64_t max_chunk = (nvec + N - 1) / N, ag_base = (int64_t)N * max_chunk;
    auto chunk_lo = [&](int c) { return nvec * c / N; };
    auto cslice = [&](int c, int64_t& lo, int64_t& hi) { slice(chunk_lo(c), chunk_lo(c + 1) - chunk_lo(c), lo, hi); };
    for (int s = 1; s < N; ++s) {  // step A
      const int q = (me + s) % N;
      int64_t lo, hi;
      cslice(q, lo, hi);
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)(me * max_chunk + (i - chunk_lo(q)))], in(i));
    }
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    {  // step B
      int64_t lo, hi;
      cslice(me, lo, hi);
      for (int64_t i = lo; i < hi; ++i) {
        uint32_t sum = 0, expect = 0;
        for (int r = 0; r < N; ++r) {
          sum += (r == me) ? in(i) : get(mine.staging[(size_t)(r * max_chunk + (i - chunk_lo(me)))]);
          expect += Model::input(k, r, i);
        }
        if (sum != expect) ++bad;
        for (int q = 0; q < N; ++q)
          if (q != me) put(m.mem[q]->staging[(size_t)(ag_base + i)], sum);
      }
    }
    signal(1, all_peers());
    if (!wait_phase(1, all_peers())) return false;
    if (me == m.slow_rank) std::this_thread::sleep_for(std::chrono::milliseconds(15));  // adversarial delay
    for (int s = 1; s < N; ++s) {  // step C
      const int q = (me + s) % N;
      int64_t lo, hi;
      cslice(q, lo, hi);
      for (int64_t i = lo; i < hi; ++i) {
        uint32_t expect = 0;
        for (int r = 0; r < N; ++r) expect += Model::input(k, r, i);
        if (get(mine.staging[(size_t)(ag_base + i)]) != expect) ++bad;
      }
    }
    return true;
  }

  // all-gather (stride 0) / all-to-all (stride 1) through staging
  bool exchange(int64_t cvec, int stride) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    for (int s = 1; s < N; ++s) {
      const int q = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)(me * cvec + i)], in((int64_t)stride * q * cvec + i));
    }
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int s = 1; s < N; ++s) {
      const int r = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i)
        if (get(mine.staging[(size_t)(r * cvec + i)]) != Model::input(k, r, (int64_t)stride * me * cvec + i)) ++bad;
    }
    return true;
  }

  // all-gather straight into every rank's peer-visible output
  bool exchange_sym(int64_t cvec) {
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    for (int s = 0; s < N; ++s) {
      const int q = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->sym[(size_t)(me * cvec + i)], in(i));
    }
    signal(1, all_peers());
    if (!wait_phase(1, all_peers())) return false;
    jitter(20);
    for (int r = 0; r < N; ++r)
      for (int64_t i = lo; i < hi; ++i)
        if (get(mine.sym[(size_t)(r * cvec + i)]) != Model::input(k, r, i)) ++bad;
    return true;
  }

  bool reduce_scatter(int64_t cvec) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    for (int s = 1; s < N; ++s) {
      const int q = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)(me * cvec + i)], in((int64_t)q * cvec + i));
    }
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int64_t i = lo; i < hi; ++i) {
      uint32_t sum = 0, expect = 0;
      for (int r = 0; r < N; ++r) {
        sum += (r == me) ? in((int64_t)me * cvec + i) : get(mine.staging[(size_t)(r * cvec + i)]);
        expect += Model::input(k, r, (int64_t)me * cvec + i);
      }
      if (sum != expect) ++bad;
    }
    return true;
  }

  // reduce-scatter that loads chunk `me` of every rank's peer-visible input
  bool reduce_scatter_sym(int64_t cvec) {
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    // the input is complete before the kernel starts; here block b provides slice b of every chunk
    for (int c = 0; c < N; ++c)
      for (int64_t i = lo; i < hi; ++i) put(mine.sym[(size_t)(c * cvec + i)], in((int64_t)c * cvec + i));
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int64_t i = lo; i < hi; ++i) {
      uint32_t sum = 0, expect = 0;
      for (int r = 0; r < N; ++r) {
        sum += get(m.mem[r]->sym[(size_t)(me * cvec + i)]);
        expect += Model::input(k, r, (int64_t)me * cvec + i);
      }
      if (sum != expect) ++bad;
    }
    signal(1, all_peers());
    return wait_phase(1, all_peers());
  }

  bool broadcast_direct(int64_t nvec, int root) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, nvec, lo, hi);
    if (me == root) {
      for (int s = 1; s < N; ++s) {
        const int q = (me + s) % N;
        for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)i], in(i));
      }
      signal(0, all_peers());
    } else {
      if (!wait_phase(0, 1u << root)) return false;
      jitter(20);
      for (int64_t i = lo; i < hi; ++i)
        if (get(mine.staging[(size_t)i]) != Model::input(k, root, i)) ++bad;
    }
    return true;
  }

  bool broadcast_twophase(int64_t nvec, int root) {
    if (!wait_prev_done()) return false;
    auto chunk_lo = [&](int c) { return nvec * c / N; };
    auto cslice = [&](int c, int64_t& lo, int64_t& hi) { slice(chunk_lo(c), chunk_lo(c + 1) - chunk_lo(c), lo, hi); };
    if (me == root) {
      for (int s = 1; s < N; ++s) {
        const int q = (me + s) % N;
        int64_t lo, hi;
        cslice(q, lo, hi);
        for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)i], in(i));
        cslice(root, lo, hi);
        for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)i], in(i));
      }
      signal(0, all_peers());
      return true;
    }
    const uint32_t others = all_peers() & ~(1u << root);
    if (!wait_phase(0, 1u << root)) return false;
    {
      int64_t lo, hi;
      cslice(me, lo, hi);
      for (int s = 1; s < N; ++s) {
        const int q = (me + s) % N;
        if (q == root) continue;
        for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)i], get(mine.staging[(size_t)i]));
      }
    }
    signal(1, others);
    if (!wait_phase(1, others)) return false;
    jitter(20);
    for (int c = 0; c < N; ++c) {
      int64_t lo, hi;
      cslice(c, lo, hi);
      for (int64_t i = lo; i < hi; ++i)
        if (get(mine.staging[(size_t)i]) != Model::input(k, root, i)) ++bad;
    }
    return true;
  }

  bool barrier() {
    signal(0, all_peers());
    return wait_phase(0, all_peers());
  }

  bool scatter(int64_t cvec, int root) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    if (me == root) {
      for (int s = 1; s < N; ++s) {
        const int q = (me + s) % N;
        for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)i], in((int64_t)q * cvec + i));
      }
      signal(0, all_peers());
      return true;
    }
    if (!wait_phase(0, 1u << root)) return false;
    jitter(20);
    for (int64_t i = lo; i < hi; ++i)
      if (get(mine.staging[(size_t)i]) != Model::input(k, root, (int64_t)me * cvec + i)) ++bad;
    return true;
  }

  bool gather(int64_t cvec, int root) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, cvec, lo, hi);
    if (me != root) {
      for (int64_t i = lo; i < hi; ++i) put(m.mem[root]->staging[(size_t)(me * cvec + i)], in(i));
      signal(0, 1u << root);
      return true;
    }
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int s = 1; s < N; ++s) {
      const int r = (me + s) % N;
      for (int64_t i = lo; i < hi; ++i)
        if (get(mine.staging[(size_t)(r * cvec + i)]) != Model::input(k, r, i)) ++bad;
    }
    return true;
  }

  bool reduce_direct(int64_t nvec, int root) {
    if (!wait_prev_done()) return false;
    int64_t lo, hi;
    slice(0, nvec, lo, hi);
    if (me != root) {
      for (int64_t i = lo; i < hi; ++i) put(m.mem[root]->staging[(size_t)(me * nvec + i)], in(i));
      signal(0, 1u << root);
      return true;
    }
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    for (int64_t i = lo; i < hi; ++i) {
      uint32_t sum = 0, expect = 0;
      for (int r = 0; r < N; ++r) {
        sum += (r == me) ? in(i) : get(mine.staging[(size_t)(r * nvec + i)]);
        expect += Model::input(k, r, i);
      }
      if (sum != expect) ++bad;
    }
    return true;
  }

  bool reduce_twophase(int64_t nvec, int root) {
    if (!wait_prev_done()) return false;
    const int64_t max_chunk = (nvec + N - 1) / N, ag_base = (int64_t)N * max_chunk;
    auto chunk_lo = [&](int c) { return nvec * c / N; };
    auto cslice = [&](int c, int64_t& lo, int64_t& hi) { slice(chunk_lo(c), chunk_lo(c + 1) - chunk_lo(c), lo, hi); };
    for (int s = 1; s < N; ++s) {
      const int q = (me + s) % N;
      int64_t lo, hi;
      cslice(q, lo, hi);
      for (int64_t i = lo; i < hi; ++i) put(m.mem[q]->staging[(size_t)(me * max_chunk + (i - chunk_lo(q)))], in(i));
    }
    signal(0, all_peers());
    if (!wait_phase(0, all_peers())) return false;
    jitter(20);
    {
      int64_t lo, hi;
      cslice(me, lo, hi);
      for (int64_t i = lo; i < hi; ++i) {
        uint32_t sum = 0, expect = 0;
        for (int r = 0; r < N; ++r) {
          sum += (r == me) ? in(i) : get(mine.staging[(size_t)(r * max_chunk + (i - chunk_lo(me)))]);
          expect += Model::input(k, r, i);
        }
        if (sum != expect) ++bad;
        if (me != root) put(m.mem[root]->staging[(size_t)(ag_base + i)], sum);
      }
    }
    if (me != root) {
      signal(1, 1u << root);
      return true;
    }
    if (!wait_phase(1, all_peers())) return false;
    for (int s = 1; s < N; ++s) {
      const int q = (me + s) % N;
      int64_t lo, hi;
      cslice(q, lo, hi);
      for (int64_t i = lo; i < hi; ++i) {
        uint32_t expect = 0;
        for (int r = 0; r < N; ++r) expect += Model::input(k, r, i);
        if (get(mine.staging[(size_t)(ag_base + i)]) != expect) ++bad;
      }
    }
    return true;
  }

  void run(const std::vector<OpDesc>& ops) {
    for (k = 0; k < ops.size(); ++k) {
      epoch = k + 1;
      const OpDesc& d = ops[k];
      bad = 0;
      jitter(50);
      bool ok = false;
      switch (d.kind) {
        case Kind::OneShot: ok = oneshot(d.nvec); break;
        case Kind::TwoShot: ok = twoshot(d.nvec); break;
        case Kind::AllGather: ok = exchange(d.nvec, 0); break;
        case Kind::AllToAll: ok = exchange(d.nvec, 1); break;
        case Kind::ReduceScatter: ok = reduce_scatter(d.nvec); break;
        case Kind::AllGatherSym: ok = exchange_sym(d.nvec); break;
        case Kind::ReduceScatterSym: ok = reduce_scatter_sym(d.nvec); break;
        case Kind::BroadcastDirect: ok = broadcast_direct(d.nvec, d.root); break;
        case Kind::BroadcastTwoPhase: ok = broadcast_twophase(d.nvec, d.root); break;
        case Kind::Barrier: ok = barrier(); break;
        case Kind::Scatter: ok = scatter(d.nvec, d.root); break;
        case Kind::Gather: ok = gather(d.nvec, d.root); break;
        case Kind::ReduceDirect: ok = reduce_direct(d.nvec, d.root); break;
        case Kind::ReduceTwoPhase: ok = reduce_twophase(d.nvec, d.root); break;
        default: break;
      }
      if (!ok) return;
      if (bad) m.errors += bad;
      // the last block of the rank to finish tells every peer that this rank is done with the op
      if (mine.counter.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)G - 1) {
        mine.counter.store(0, std::memory_order_relaxed);
        for (int q = 0; q < N; ++q) m.mem[q]->done[me].store(epoch, std::memory_order_release);
      }
      // kernel boundary on the rank's stream: no block starts op k+1 before every block of
      // the rank has finished op k (the rank's own slot of `done` stands in for it here)
      if (!m.wait(mine.done[me], epoch)) return;
    }
  }
};

}  // namespace

ProtocolModelResult run_protocol_model(int nranks, int blocks, int n_ops, uint32_t seed, bool use_done_chain,
                                       int slow_rank, bool mix) {
  ProtocolModelResult res;
  if (nranks < 2 || nranks > 8 || blocks < 1 || blocks > 8 || n_ops < 1) {
    res.errors = 1;
    return res;
  }
  std::mt19937 rng(seed);
  std::vector<OpDesc> ops;
  int64_t max_words = 0, max_sym = 1;
  for (int k = 0; k < n_ops; ++k) {
    OpDesc d;
    d.root = (int)(rng() % (uint32_t)nranks);
    d.nvec = 32 + (int64_t)(rng() % 96);
    d.kind = (k % 2 == 1) ? Kind::OneShot : Kind::TwoShot;  // alternate layouts: consecutive ops reuse addresses differently
    if (mix) d.kind = (Kind)(rng() % (uint32_t)Kind::kCount);
    if (slow_rank >= 0) d.nvec = 64;  // sizes chosen so the two all-reduce layouts overlap exactly
    int64_t need = 0;
    switch (d.kind) {
      case Kind::OneShot: need = (int64_t)nranks * d.nvec; break;
      case Kind::TwoShot: need = (int64_t)nranks * ((d.nvec + nranks - 1) / nranks) + d.nvec; break;
      case Kind::AllGather:
      case Kind::AllToAll:
      case Kind::ReduceScatter:
        d.nvec = 3 + d.nvec / 4;  // words per chunk
        need = (int64_t)nranks * d.nvec;
        break;
      case Kind::AllGatherSym:
      case Kind::ReduceScatterSym:
        d.nvec = 3 + d.nvec / 4;
        max_sym = std::max(max_sym, (int64_t)nranks * d.nvec);
        break;
      case Kind::BroadcastDirect:
      case Kind::BroadcastTwoPhase: need = d.nvec; break;
      case Kind::Scatter:
        d.nvec = 3 + d.nvec / 4;
        need = d.nvec;
        break;
      case Kind::Gather:
        d.nvec = 3 + d.nvec / 4;
        need = (int64_t)nranks * d.nvec;
        break;
      case Kind::ReduceDirect: need = (int64_t)nranks * d.nvec; break;
      case Kind::ReduceTwoPhase: need = (int64_t)nranks * ((d.nvec + nranks - 1) / nranks) + d.nvec; break;
      default: break;
    }
    max_words = std::max(max_words, need);
    ops.push_back(d);
  }
  Model m;
  m.N = nranks;
  m.G = blocks;
  m.use_done = use_done_chain;
  m.slow_rank = slow_rank;
  for (int r = 0; r < nranks; ++r)
    m.mem.push_back(std::make_unique<RankMem>((size_t)std::max<int64_t>(max_words, 1), (size_t)max_sym, nranks, blocks));
  std::vector<std::thread> threads;
  for (int r = 0; r < nranks; ++r)
    for (int b = 0; b < blocks; ++b) threads.emplace_back([&m, r, b, &ops, seed] {
      Block blk(m, r, b, seed * 131u + (uint32_t)(r * 17 + b));
      blk.run(ops);
    });
  for (auto& t : threads) t.join();
  res.errors = m.errors.load();
  res.timeouts = m.timeouts.load();
  res.ops = (uint64_t)n_ops;
  return res;
}

}  // namespace bagua
