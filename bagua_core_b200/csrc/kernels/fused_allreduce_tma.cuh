// All-reduce on symmetric buffers with the data moved by the SM's bulk-copy engine (TMA),
// sm_100a.
//
// Why: a communication kernel that overlaps the backward pass costs the compute kernels
// roughly (SMs it occupies) x (time it stays resident).  The time is bounded below by the
// NVLink rate, so what matters is how many bytes ONE SM keeps in flight.  With ordinary loads
// that is registers: 512 threads x 8 outstanding 16-byte peer loads = 64 KB per SM, about
// 10 GB/s per SM at a loaded round trip of several microseconds, i.e. 64 SMs for the link.
// Here a few elected threads issue `cp.async.bulk` copies of whole tiles from the peers'
// buffers into a ring of shared-memory stages (128-192 KB in flight per SM, no registers
// held), the block sums the tiles out of shared memory, and the result tile leaves through
// bulk stores to every rank's output.  A dozen SMs then carry the link.
//
// Algorithm (same as allreduce_sym_body): rank r owns chunk r; block b owns slice b of it.
//   signal "my input is final" / wait for the peers' blocks b
//   for every tile of the slice, S stages deep:
//     bulk-load the tile from all N inputs         (mbarrier complete_tx per stage)
//     sum in rank order (fp32), scale              (all threads, shared memory to shared memory)
//     bulk-store the result tile to all N outputs  (bulk async-group per tile)
//   wait for the stores, signal "my stores are done" / wait for the peers'
//
// No tensor map, no cluster, no multicast: the copies are 1-D, between this block's own shared
// memory and global memory (local or a peer's).  Every wait is bounded (see peer_sync.cuh);
// when one gives up, the block stops issuing, waits (bounded again) for the loads it still has
// in flight into its shared memory, waits for its stores, and leaves through cta_finish_op.
//
// The same body compiles for the host (BAGUA_HOST_EMULATION), with the copies and mbarriers
// replaced by stand-ins that keep their counting rules, to run under the thread and address
// sanitizers (tests/cpp/device_emulation.cc).
//
// The reference has no counterpart: its all-reduce is one NCCL call
// (bagua-core-internal/src/comm_ops/centralized_full_precision_synchronous.rs:16-55).
#pragma once

#include <cuda_runtime.h>

#include "fused_allreduce_bodies.cuh"
#include "peer_sync.cuh"
#include "vec_ops.cuh"

namespace bagua {
namespace fused {
namespace allreduce_bodies {

#ifndef BAGUA_HOST_EMULATION
constexpr int kTmaThreads = 256;
constexpr int kTmaStageInBytes = 32 << 10;  // input of one stage: NR tiles of 32 KB / NR
constexpr int kTmaRingBytes = 216 << 10;    // 2 ranks: 4 stages, 4 ranks: 5, 8 ranks: 6
constexpr int kTmaMbarBytes = 8;
#else
// On the host the same body runs with one thread per CUDA thread of a one-warp block and a
// ring small enough that the few hundred bytes of a test wrap it several times.
constexpr int kTmaThreads = 32;
constexpr int kTmaStageInBytes = 256;
constexpr int kTmaRingBytes = 3 * (256 + 128);
constexpr int kTmaMbarBytes = 16;  // the host's stand-in for an mbarrier, see tma::HostMbar
#endif

template <int NR>
struct TmaCfg {
  static constexpr int kTileVecs = kTmaStageInBytes / 16 / NR;            // vectors per source tile
  static constexpr int kStageBytes = kTmaStageInBytes + kTileVecs * 16;   // N input tiles + one output tile
  static constexpr int kStages = kTmaRingBytes / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStages * kTmaMbarBytes;  // + one mbarrier per stage
};

#ifndef BAGUA_HOST_EMULATION
namespace tma {

using saddr_t = uint32_t;  // an address in this block's shared memory
using bar_t = uint32_t;    // the shared-memory address of an mbarrier
__device__ __forceinline__ bar_t bar_at(unsigned char* bars, int s) { return (uint32_t)__cvta_generic_to_shared(bars) + (uint32_t)(kTmaMbarBytes * s); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> this block's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// this block's shared memory -> global, member of the thread's current bulk async-group
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace tma
#else  // BAGUA_HOST_EMULATION
// The host's bulk-copy engine: a copy is done by the thread that issues it, at once, and then
// counted on the stage's barrier.  The barrier keeps the device's rules (one pending arrival per
// phase, a transaction count in bytes that may go negative before the arrival arms it, a phase
// that completes when both reach zero), so a body that arms too little, waits on the wrong
// parity or reuses a stage too early stalls or trips the sanitizers here as well.
namespace tma {

struct HostMbar {
  uint32_t lock;     // spin lock (acquire / release), so the sanitizers see the hand-over
  uint32_t phase;    // completed phases
  int32_t pending;   // arrivals the current phase still waits for
  int32_t tx;        // bytes the current phase still waits for
};
static_assert(sizeof(HostMbar) == kTmaMbarBytes, "size of the emulated mbarrier");
using saddr_t = unsigned char*;
using bar_t = HostMbar*;

inline bar_t bar_at(unsigned char* bars, int s) { return reinterpret_cast<HostMbar*>(bars) + s; }
inline saddr_t smem_addr(const void* p) { return static_cast<unsigned char*>(const_cast<void*>(p)); }
inline void mbar_lock(bar_t b) {
  while (__atomic_exchange_n(&b->lock, 1u, __ATOMIC_ACQUIRE) != 0) sched_yield();
}
inline void mbar_unlock(bar_t b) { __atomic_store_n(&b->lock, 0u, __ATOMIC_RELEASE); }
inline void mbar_settle(bar_t b, int32_t count) {  // under the lock
  if (b->pending == 0 && b->tx == 0) {
    b->phase += 1;
    b->pending = count;
  }
}
inline void mbar_init(bar_t b, uint32_t count) {
  b->phase = 0;
  b->pending = (int32_t)count;
  b->tx = 0;
  __atomic_store_n(&b->lock, 0u, __ATOMIC_RELEASE);
}
inline void fence_mbar_init() {}
inline void mbar_expect_tx(bar_t b, uint32_t bytes) {
  mbar_lock(b);
  b->tx += (int32_t)bytes;
  b->pending -= 1;
  mbar_settle(b, 1);
  mbar_unlock(b);
}
inline bool mbar_try_wait(bar_t b, uint32_t parity) {
  mbar_lock(b);
  const bool done = (b->phase & 1u) != parity;
  mbar_unlock(b);
  return done;
}
inline void bulk_load(saddr_t dst, const void* src, uint32_t bytes, bar_t b) {
  std::memcpy(dst, src, bytes);
  mbar_lock(b);
  b->tx -= (int32_t)bytes;
  mbar_settle(b, 1);
  mbar_unlock(b);
}
inline void bulk_store(void* dst, saddr_t src, uint32_t bytes) { std::memcpy(dst, src, bytes); }
inline void bulk_commit() {}
template <int N>
inline void bulk_wait_read() {}
inline void bulk_wait_all() {}
inline void fence_proxy_async() {}
inline void fence_proxy_async_smem() {}

}  // namespace tma
#endif

namespace tma {
// One thread waits for phase `parity` of `bar`; bounded like every other wait.  Status code 5.
__device__ __forceinline__ bool mbar_wait(const ArenaView& v, const Launch& L, bar_t bar, uint32_t parity,
                                          uint32_t stage) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t* poison = v.signals[v.rank] + kSigPoison;
  const uint64_t start = psync::globaltimer_ns();
  const uint64_t max_spins = v.deadline_ns / 64 + (1ull << 20);
  for (uint64_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 31) == 0) {
      if (psync::ld_relaxed_gpu(poison) != 0) return false;
      if (psync::globaltimer_ns() - start > v.deadline_ns || spins > max_spins) {
        psync::record_timeout(v, 5, stage, (uint32_t)v.rank, parity, (uint32_t)L.block);
        return false;
      }
    }
  }
}

}  // namespace tma

// `smem` is the kernel's dynamic shared memory (TmaCfg<NR>::kSmemBytes, 128-byte aligned).
template <typename T, int NR>
__device__ __forceinline__ void allreduce_sym_tma_body(const ArenaView& v, const Launch& L, const SymPtrs& p,
                                                       int64_t nvec, float scale, unsigned char* smem) {
  using O = VecOps<T>;
  using C = TmaCfg<NR>;
  constexpr int S = C::kStages, TV = C::kTileVecs;
  const int me = v.rank, tid = threadIdx.x;
  const int G = L.grid, b = L.block;
  const int64_t c0 = nvec * me / NR, len = nvec * (me + 1) / NR - c0;
  const int64_t lo = c0 + len * b / G, hi = c0 + len * (b + 1) / G;
  const int64_t ntiles = (hi - lo + TV - 1) / TV;

  uint4* in_s = reinterpret_cast<uint4*>(smem);                                     // [S][NR][TV]
  uint4* out_s = reinterpret_cast<uint4*>(smem + (size_t)S * kTmaStageInBytes);      // [S][TV]
  unsigned char* bars = smem + (size_t)S * C::kStageBytes;                          // [S] mbarriers
  const tma::saddr_t in0 = tma::smem_addr(in_s), out0 = tma::smem_addr(out_s);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) tma::mbar_init(tma::bar_at(bars, s), 1);
    tma::fence_mbar_init();
  }
  // first signal: every peer's block b has started, i.e. that peer's input is final
  psync::cta_signal_phase(v, L, 0, all_peers_mask(v));
  bool ok = psync::cta_wait_phase(v, L, 0, all_peers_mask(v));

  auto tile_vecs = [&](int64_t k) {
    const int64_t left = hi - (lo + k * TV);
    return (int)(left < TV ? left : TV);
  };
  // Lanes 0 .. NR-1 of warp 0 are the issuers: lane r moves rank r's tiles (its loads and the
  // stores into rank r's output form that lane's own bulk async-groups), so the NR copies of a
  // tile are issued side by side instead of one after the other.  Lane 0 also arms the stage's
  // mbarrier; the phase cannot complete before that arrival, whichever lane's bytes land first.
  const bool issuer = tid < NR;
  auto issue_load = [&](int64_t k) {  // issuers
    const int s = (int)(k % S);
    const uint32_t bytes = (uint32_t)tile_vecs(k) * 16u;
    if (tid == 0) tma::mbar_expect_tx(tma::bar_at(bars, s), bytes * NR);
    tma::bulk_load(in0 + (uint32_t)((s * NR + tid) * TV) * 16u, p.in[tid] + lo + k * TV, bytes, tma::bar_at(bars, s));
  };

  int64_t issued = 0;  // tiles whose loads have been issued (the same in every issuer)
  if (ok && issuer) {
    tma::fence_proxy_async();  // the peers' inputs, acquired through generic-proxy loads, are read by the copy engine
    for (; issued < ntiles && issued < S; ++issued) issue_load(issued);
  }
  int64_t k = 0;
  if (ok) {
    for (; k < ntiles; ++k) {
      const int s = (int)(k % S);
      // everyone waits for the stage: the mbarrier's completion is what makes the copied bytes visible
      bool got = tma::mbar_wait(v, L, tma::bar_at(bars, s), (uint32_t)((k / S) & 1), (uint32_t)s);
      // the stores that last read out_s[s] (tile k - S) must have left shared memory
      if (issuer && k >= S) tma::bulk_wait_read<S - 1>();
      if (!__syncthreads_and(got)) {
        ok = false;
        break;
      }
      const int tv = tile_vecs(k);
      const uint4* src = in_s + (size_t)s * NR * TV;
      uint4* dst = out_s + (size_t)s * TV;
      for (int j = tid; j < tv; j += kTmaThreads) {
        float a[O::N];
#pragma unroll
        for (int e = 0; e < O::N; ++e) a[e] = 0.f;
#pragma unroll
        for (int r = 0; r < NR; ++r) O::acc(a, src[r * TV + j]);
        dst[j] = O::pack(a, scale);
      }
      tma::fence_proxy_async_smem();  // my shared-memory stores, before the copy engine reads them
      __syncthreads();                // all of out_s[s] written, all of in_s[s] read
      if (issuer) {
        tma::bulk_store(p.out[tid] + lo + k * TV, out0 + (uint32_t)(s * TV) * 16u, (uint32_t)tv * 16u);
        tma::bulk_commit();
        if (issued < ntiles) issue_load(issued++);
      }
    }
  }
  // Leaving early: loads that were issued for tiles k.. are still landing in this block's shared
  // memory; the thread that issued them waits for them (bounded again) before anyone returns.
  if (!ok) {
    if (tid == 0)  // lane 0 issued as many tiles as every other issuer
      for (int64_t q = k; q < issued; ++q)
        tma::mbar_wait(v, L, tma::bar_at(bars, (int)(q % S)), (uint32_t)((q / S) & 1), (uint32_t)(q % S));
    __syncthreads();
  }
  if (issuer) {
    tma::bulk_wait_all();      // this lane's result tiles have been written to its rank's output
    tma::fence_proxy_async();  // ... and are ordered before the generic-proxy release below
  }
  if (ok) {
    // second signal: my stores into everyone's output are complete / theirs into mine
    psync::cta_signal_phase(v, L, 1, all_peers_mask(v));
    ok = psync::cta_wait_phase(v, L, 1, all_peers_mask(v));
  }
  psync::cta_finish_op(v, L);
}

}  // namespace allreduce_bodies
}  // namespace fused
}  // namespace bagua
