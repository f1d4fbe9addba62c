// Device-side signalling between GPUs for the fused communication kernels.
//
// Memory model: a producer CTA writes payload with ordinary stores to a peer pointer,
// executes bar.sync, then one thread issues fence.sys + st.release.sys on the peer's
// signal word.  The consumer thread polls the word with ld.acquire.sys, then bar.sync
// releases the rest of its CTA, which may now read the payload.  Signal values are op
// epochs that only grow (compared with wrap-around arithmetic).
//
// Every wait is bounded twice: by %globaltimer against the view's deadline and by an
// iteration cap.  When a wait runs out the thread records what it was waiting for in
// the host-mapped status record, raises the rank-local poison word so that all other
// waits on this GPU return at once, and gives up; no trap, no assert.
//
// `Launch` is the block's position inside its rank's grid.  In a real launch it is
// {blockIdx.x, gridDim.x}.  The single-GPU emulation (one cooperative launch that hosts
// the grids of all ranks side by side, for tests on a machine with fewer GPUs than
// ranks) passes the position inside the virtual rank instead.
#pragma once

#include <cuda_runtime.h>

#include "../comm/arena.h"
#include "host_emulation.h"

namespace bagua {
namespace psync {

using bagua::kSigPoison;  // rank-local: non-zero once any wait ran out, or the host aborted the communicator

struct Launch {
  int block;  // index of this block inside its rank's grid
  int grid;   // number of blocks of its rank's grid
};
__device__ __forceinline__ Launch real_launch() { return Launch{(int)blockIdx.x, (int)gridDim.x}; }

#ifdef BAGUA_HOST_EMULATION
// The same five primitives for the host-thread emulation of the device code.
inline uint64_t globaltimer_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
inline void st_release_sys(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline uint32_t ld_acquire_sys(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline uint32_t ld_relaxed_gpu(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
inline uint64_t ld_acquire_gpu_u64(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
#else
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
#endif

__device__ __forceinline__ uint32_t* phase_word(uint32_t* pad, int phase, int src, int block) {
  return pad + kSigPhase + (phase * kArenaMaxRanks + src) * kArenaMaxBlocks + block;
}

static __device__ __noinline__ void record_timeout(const ArenaView& v, uint32_t code, uint32_t phase, uint32_t peer,
                                                   uint32_t seen, uint32_t block) {
  DeviceStatus* s = v.status;
  if (s) {
    volatile uint32_t* w = reinterpret_cast<volatile uint32_t*>(s);
    w[1] = phase;
    w[2] = peer;
    w[3] = block;
    w[4] = v.epoch;
    w[5] = seen;
    __threadfence_system();
    w[0] = code;
  }
  volatile uint32_t* poison = v.signals[v.rank] + kSigPoison;
  *poison = 1u;
  __threadfence();
}

// One thread waits until *flag has reached `want`.  Returns false when it gave up.
__device__ __forceinline__ bool wait_word(const ArenaView& v, const Launch& L, const uint32_t* flag, uint32_t want,
                                          uint32_t code, uint32_t phase, uint32_t peer) {
  uint32_t seen = ld_acquire_sys(flag);
  if ((int32_t)(seen - want) >= 0) return true;
  const uint32_t* poison = v.signals[v.rank] + kSigPoison;
  const uint64_t start = globaltimer_ns();
  const uint64_t max_spins = v.deadline_ns / 64 + (1ull << 20);
  for (uint64_t spins = 1;; ++spins) {
    seen = ld_acquire_sys(flag);
    if ((int32_t)(seen - want) >= 0) return true;
    if ((spins & 31) == 0) {
      if (ld_relaxed_gpu(poison) != 0) return false;
      if (globaltimer_ns() - start > v.deadline_ns || spins > max_spins) {
        record_timeout(v, code, phase, peer, seen, (uint32_t)L.block);
        return false;
      }
      if (spins > 4096) __nanosleep(200);
    }
  }
}

// CTA-wide: wait until every peer's previous fused op has finished (its `done` word
// reached epoch-1).  All threads must call.  Returns false if any wait gave up.
__device__ __forceinline__ bool cta_wait_prev_done(const ArenaView& v, const Launch& L) {
  bool ok = true;
  const int t = threadIdx.x;
  if (t < v.nranks && t != v.rank) ok = wait_word(v, L, v.signals[v.rank] + kSigDone + t, v.epoch - 1, 1, 0, t);
  return __syncthreads_and(ok) != 0;
}

// CTA-wide: publish "this block finished writing phase `phase` data" to every peer in
// `peer_mask` (bit q).  All threads must call; payload stores must precede the call.
__device__ __forceinline__ void cta_signal_phase(const ArenaView& v, const Launch& L, int phase, uint32_t peer_mask) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < v.nranks && ((peer_mask >> t) & 1u)) {
    __threadfence_system();
    st_release_sys(phase_word(v.signals[t], phase, v.rank, L.block), v.epoch);
  }
}

// CTA-wide: wait for block `L.block` of every peer in `peer_mask` to have published
// phase `phase`.  Returns false if any wait gave up.
__device__ __forceinline__ bool cta_wait_phase(const ArenaView& v, const Launch& L, int phase, uint32_t peer_mask) {
  bool ok = true;
  const int t = threadIdx.x;
  if (t < v.nranks && ((peer_mask >> t) & 1u))
    ok = wait_word(v, L, phase_word(v.signals[v.rank], phase, t, L.block), v.epoch, 2, phase, t);
  return __syncthreads_and(ok) != 0;
}

// CTA-wide, at the very end of a fused op: the last CTA of the rank's grid tells every
// peer that this rank is done with the op (so they may overwrite its staging next op).
__device__ __forceinline__ void cta_finish_op(const ArenaView& v, const Launch& L) {
  __syncthreads();
  BAGUA_SHARED(int, s_last, 0);
  uint32_t* pad = v.signals[v.rank];
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(pad + kSigCounter, 1u);
    s_last = (prev == (uint32_t)L.grid - 1);
    if (s_last) pad[kSigCounter] = 0u;  // ready for the next launch (stream-ordered)
  }
  __syncthreads();
  if (s_last) {
    const int t = threadIdx.x;
    if (t < v.nranks && t != v.rank) {
      __threadfence_system();
      st_release_sys(v.signals[t] + kSigDone + v.rank, v.epoch);
    }
  }
}

// Barrier over the rank's grid on a rank-local 64-bit counter that only grows; `index`
// is the barrier's ordinal inside this launch (0, 1, ...).  Needs all CTAs co-resident
// (cooperative launch).  Returns false if the wait gave up.
__device__ __forceinline__ bool grid_barrier(const ArenaView& v, const Launch& L, int index) {
  __syncthreads();
  BAGUA_SHARED(int, s_ok, 1);
  if (threadIdx.x == 0) {
    unsigned long long* ctr = reinterpret_cast<unsigned long long*>(v.signals[v.rank] + kSigGridBar);
    const unsigned long long target = v.grid_bar_base + (unsigned long long)(index + 1) * (unsigned long long)L.grid;
    __threadfence();
    atomicAdd(ctr, 1ull);
    bool ok = true;
    const uint32_t* poison = v.signals[v.rank] + kSigPoison;
    const uint64_t start = globaltimer_ns();
    const uint64_t max_spins = v.deadline_ns / 64 + (1ull << 20);
    for (uint64_t spins = 1; ld_acquire_gpu_u64(ctr) < target; ++spins) {
      if ((spins & 31) == 0) {
        if (ld_relaxed_gpu(poison) != 0) {
          ok = false;
          break;
        }
        if (globaltimer_ns() - start > v.deadline_ns || spins > max_spins) {
          record_timeout(v, 3, (uint32_t)index, 0, 0, (uint32_t)L.block);
          ok = false;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace psync
}  // namespace bagua
