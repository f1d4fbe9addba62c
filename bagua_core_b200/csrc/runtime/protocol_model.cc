// Host-thread model of the cross-GPU signalling protocol used by the fused kernels.
//
// compute-sanitizer cannot be run on the GPU pool, so the protocol (epoch-valued phase
// words, the `done` chain that guards staging reuse, block-to-block pairing) is restated
// here with std::thread + std::atomic and the same acquire/release structure, and run
// under randomised and adversarial schedules:
//   * every (rank, block) pair is a thread; payload words are relaxed atomics (the GPU's
//     weak accesses), signal words use release stores / acquire loads;
//   * a run is a sequence of all-reduces that mixes the one-shot and the two-shot layout,
//     so consecutive ops reuse the same staging addresses for different purposes;
//   * inputs depend on (op, rank, index): any premature overwrite or stale read shows up
//     as a wrong sum; every wait is bounded and counted when it runs out.
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

struct RankMem {
  std::vector<std::atomic<uint32_t>> staging;
  std::vector<std::atomic<uint32_t>> done;    // [nranks]
  std::vector<std::atomic<uint32_t>> phase;   // [2][nranks][blocks]
  std::atomic<uint32_t> counter{0};
  std::vector<uint32_t> data;                 // the rank's bucket (only its own threads touch it)
  RankMem(size_t stage_words, int nranks, int blocks)
      : staging(stage_words), done((size_t)nranks), phase((size_t)2 * nranks * blocks) {
    for (auto& a : staging) a.store(0xdeadbeefu);
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
  int64_t nvec;
  bool oneshot;
};

void block_thread(Model& m, int me, int b, const std::vector<OpDesc>& ops, uint32_t seed) {
  std::mt19937 rng(seed);
  auto jitter = [&](int max_us) {
    if (max_us > 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % (uint32_t)max_us));
  };
  const int N = m.N, G = m.G;
  RankMem& mine = *m.mem[me];
  for (uint32_t k = 0; k < ops.size(); ++k) {
    const uint32_t epoch = k + 1;
    const int64_t nvec = ops[k].nvec;
    // the bucket of this op (block 0 of each rank fills it; others wait for it via the counter trick
    // of a real launch: here every block simply fills its own slice before use)
    auto in = [&](int64_t i) { return Model::input(k, me, i); };
    jitter(50);
    // wait for the peers' previous op to be completely finished
    if (m.use_done)
      for (int q = 0; q < N; ++q)
        if (q != me && !m.wait(mine.done[q], epoch - 1)) return;
    uint64_t bad = 0;
    if (ops[k].oneshot) {
      const int64_t lo = nvec * b / G, hi = nvec * (b + 1) / G;
      for (int s = 1; s < N; ++s) {
        const int q = (me + s) % N;
        for (int64_t i = lo; i < hi; ++i)
          m.mem[q]->staging[(size_t)me * nvec + i].store(in(i), std::memory_order_relaxed);
      }
      for (int q = 0; q < N; ++q)
        if (q != me) m.phase(q, 0, me, b).store(epoch, std::memory_order_release);
      for (int q = 0; q < N; ++q)
        if (q != me && !m.wait(m.phase(me, 0, q, b), epoch)) return;
      jitter(20);
      for (int64_t i = lo; i < hi; ++i) {
        uint32_t sum = 0, expect = 0;
        for (int r = 0; r < N; ++r) {
          sum += (r == me) ? in(i) : mine.staging[(size_t)r * nvec + i].load(std::memory_order_relaxed);
          expect += Model::input(k, r, i);
        }
        if (sum != expect) ++bad;
      }
    } else {
      const int64_t max_chunk = (nvec + N - 1) / N, ag_base = (int64_t)N * max_chunk;
      auto chunk_lo = [&](int c) { return nvec * c / N; };
      auto slice = [&](int c, int64_t& lo, int64_t& hi) {
        const int64_t c0 = chunk_lo(c), len = chunk_lo(c + 1) - c0;
        lo = c0 + len * b / G;
        hi = c0 + len * (b + 1) / G;
      };
      for (int s = 1; s < N; ++s) {  // step A
        const int q = (me + s) % N;
        int64_t lo, hi;
        slice(q, lo, hi);
        for (int64_t i = lo; i < hi; ++i)
          m.mem[q]->staging[(size_t)(me * max_chunk + (i - chunk_lo(q)))].store(in(i), std::memory_order_relaxed);
      }
      for (int q = 0; q < N; ++q)
        if (q != me) m.phase(q, 0, me, b).store(epoch, std::memory_order_release);
      for (int q = 0; q < N; ++q)
        if (q != me && !m.wait(m.phase(me, 0, q, b), epoch)) return;
      jitter(20);
      {  // step B
        int64_t lo, hi;
        slice(me, lo, hi);
        for (int64_t i = lo; i < hi; ++i) {
          uint32_t sum = 0, expect = 0;
          for (int r = 0; r < N; ++r) {
            sum += (r == me) ? in(i)
                             : mine.staging[(size_t)(r * max_chunk + (i - chunk_lo(me)))].load(std::memory_order_relaxed);
            expect += Model::input(k, r, i);
          }
          if (sum != expect) ++bad;
          for (int q = 0; q < N; ++q)
            if (q != me) m.mem[q]->staging[(size_t)(ag_base + i)].store(sum, std::memory_order_relaxed);
        }
      }
      for (int q = 0; q < N; ++q)
        if (q != me) m.phase(q, 1, me, b).store(epoch, std::memory_order_release);
      for (int q = 0; q < N; ++q)
        if (q != me && !m.wait(m.phase(me, 1, q, b), epoch)) return;
      if (me == m.slow_rank) std::this_thread::sleep_for(std::chrono::milliseconds(15));  // adversarial delay
      for (int s = 1; s < N; ++s) {  // step C
        const int q = (me + s) % N;
        int64_t lo, hi;
        slice(q, lo, hi);
        for (int64_t i = lo; i < hi; ++i) {
          uint32_t expect = 0;
          for (int r = 0; r < N; ++r) expect += Model::input(k, r, i);
          if (mine.staging[(size_t)(ag_base + i)].load(std::memory_order_relaxed) != expect) ++bad;
        }
      }
    }
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

}  // namespace

ProtocolModelResult run_protocol_model(int nranks, int blocks, int n_ops, uint32_t seed, bool use_done_chain,
                                       int slow_rank) {
  ProtocolModelResult res;
  if (nranks < 2 || nranks > 8 || blocks < 1 || blocks > 8 || n_ops < 1) {
    res.errors = 1;
    return res;
  }
  std::mt19937 rng(seed);
  std::vector<OpDesc> ops;
  int64_t max_words = 0;
  for (int k = 0; k < n_ops; ++k) {
    OpDesc d;
    d.nvec = 32 + (int64_t)(rng() % 96);
    d.oneshot = (k % 2 == 1);  // alternate layouts so that consecutive ops reuse addresses differently
    if (slow_rank >= 0) d.nvec = 64;  // sizes chosen so the two layouts overlap exactly
    const int64_t need = d.oneshot ? (int64_t)nranks * d.nvec : (int64_t)nranks * ((d.nvec + nranks - 1) / nranks) + d.nvec;
    max_words = std::max(max_words, need);
    ops.push_back(d);
  }
  Model m;
  m.N = nranks;
  m.G = blocks;
  m.use_done = use_done_chain;
  m.slow_rank = slow_rank;
  for (int r = 0; r < nranks; ++r) m.mem.push_back(std::make_unique<RankMem>((size_t)max_words, nranks, blocks));
  // a rank's own `done` word doubles as its kernel boundary: set by its last block
  std::vector<std::thread> threads;
  for (int r = 0; r < nranks; ++r)
    for (int b = 0; b < blocks; ++b) threads.emplace_back([&m, r, b, &ops, seed] {
      // wrap: make the rank's last-block signal also visible to its own blocks
      block_thread(m, r, b, ops, seed * 131u + (uint32_t)(r * 17 + b));
    });
  for (auto& t : threads) t.join();
  res.errors = m.errors.load();
  res.timeouts = m.timeouts.load();
  res.ops = (uint64_t)n_ops;
  return res;
}

}  // namespace bagua
