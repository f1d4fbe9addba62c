// Host stand-ins for the CUDA device environment, so that the `*_body` device functions of
// the fused communication kernels can be compiled by the host compiler and run as ordinary
// threads: one OS thread per CUDA thread, a std::barrier per block, per-block storage for
// `__shared__` variables, and GCC atomics in place of the PTX memory-model instructions
// (st.release.sys → release store, ld.acquire.sys → acquire load, fence.sys → seq_cst fence).
// Payload accesses stay plain loads and stores, exactly as on the device, which is what lets
// ThreadSanitizer check that the signalling protocol orders them.
//
// Only active with -DBAGUA_HOST_EMULATION (tests/cpp/device_emulation.cc); a device build
// never sees this file's contents.
#pragma once

#ifdef BAGUA_HOST_EMULATION

#include <cuda_runtime.h>  // vector types (uint4, make_uint4) and empty __device__ / __forceinline__ on the host
#include <sched.h>
#include <time.h>

#include <barrier>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

namespace bagua {
namespace hostemu {

// One per emulated block; every thread of the block points at it.
struct BlockContext {
  explicit BlockContext(int threads) : nthreads(threads), bar(threads) {}
  int nthreads;
  std::barrier<> bar;
  int vote = 1;               // accumulator of __syncthreads_and
  alignas(16) char shared[256] = {};  // storage of BAGUA_SHARED variables, by slot
  float lanes[32] = {};       // exchange buffer of the warp shuffles (a block is one warp)
  std::mutex arrays_mu;
  std::map<int, std::vector<uint64_t>> arrays;  // storage of BAGUA_SHARED_ARRAY variables, by slot

  void* array(int slot, size_t bytes) {
    std::lock_guard<std::mutex> g(arrays_mu);
    auto& a = arrays[slot];
    if (a.size() * 8 < bytes) a.resize((bytes + 7) / 8);
    return a.data();
  }
};

struct Dim {
  unsigned x = 0, y = 0, z = 0;
};

inline thread_local BlockContext* t_block = nullptr;
inline thread_local Dim t_thread_idx;
inline thread_local Dim t_block_idx;
inline thread_local Dim t_grid_dim;
inline thread_local Dim t_block_dim;

inline void bind_thread(BlockContext* b, unsigned tid, unsigned block, unsigned grid) {
  t_block = b;
  t_thread_idx.x = tid;
  t_block_idx.x = block;
  t_grid_dim.x = grid;
  t_block_dim.x = (unsigned)b->nthreads;
}

inline void syncthreads() { t_block->bar.arrive_and_wait(); }

inline int syncthreads_and(int pred) {
  BlockContext* b = t_block;
  b->bar.arrive_and_wait();  // everyone has read the previous vote's result
  if (t_thread_idx.x == 0) __atomic_store_n(&b->vote, 1, __ATOMIC_RELAXED);
  b->bar.arrive_and_wait();
  if (!pred) __atomic_store_n(&b->vote, 0, __ATOMIC_RELAXED);
  b->bar.arrive_and_wait();
  return __atomic_load_n(&b->vote, __ATOMIC_RELAXED);
}

template <typename T>
inline T& shared_slot(int slot) {
  static_assert(sizeof(T) <= 16, "a shared slot holds 16 bytes");
  return *reinterpret_cast<T*>(t_block->shared + 16 * slot);
}

template <typename T>
inline T* shared_array(int slot, size_t count) {
  return static_cast<T*>(t_block->array(slot, count * sizeof(T)));
}

// __shfl_xor_sync for a block that is exactly one warp and in which every thread takes part:
// everyone publishes its value, reads its partner's, and waits until all have read.
inline float shfl_xor(float v, int lane_mask) {
  BlockContext* b = t_block;
  const unsigned me = t_thread_idx.x;
  b->lanes[me] = v;
  b->bar.arrive_and_wait();
  const float r = b->lanes[(me ^ (unsigned)lane_mask) % (unsigned)b->nthreads];
  b->bar.arrive_and_wait();
  return r;
}

}  // namespace hostemu
}  // namespace bagua

#define threadIdx (::bagua::hostemu::t_thread_idx)
#define blockIdx (::bagua::hostemu::t_block_idx)
#define gridDim (::bagua::hostemu::t_grid_dim)
#define blockDim (::bagua::hostemu::t_block_dim)
#define __shfl_xor_sync(mask, v, lane_mask) ::bagua::hostemu::shfl_xor((v), (lane_mask))
#define __syncthreads() ::bagua::hostemu::syncthreads()
#define __syncthreads_and(p) ::bagua::hostemu::syncthreads_and((p) ? 1 : 0)
// ThreadSanitizer does not model stand-alone fences.  The protocol never relies on one for
// ordering between threads here (every hand-over is a release store / acquire load on a signal
// word plus a block barrier), so under the sanitizer the fences compile to nothing.
#if defined(__SANITIZE_THREAD__)
#define __threadfence() ((void)0)
#define __threadfence_system() ((void)0)
#else
#define __threadfence() __atomic_thread_fence(__ATOMIC_SEQ_CST)
#define __threadfence_system() __atomic_thread_fence(__ATOMIC_SEQ_CST)
#endif
#define __nanosleep(ns) sched_yield()
#ifndef __noinline__
#define __noinline__ __attribute__((noinline))
#endif

inline uint32_t atomicAdd(uint32_t* p, uint32_t v) { return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL); }
inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v) {
  return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL);
}
inline float __uint_as_float(unsigned u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline unsigned __float_as_uint(float f) {
  unsigned u;
  std::memcpy(&u, &f, 4);
  return u;
}

// Chunk headers are written by every block of a rank with the same value, and a peer may read
// one while a later block of the writer stores it again.  On the device these are plain word
// accesses (one aligned word, same bits every time); here they are relaxed atomics, so that
// ThreadSanitizer accepts exactly this pattern and nothing else.
namespace bagua {
template <typename T>
inline void same_value_store(T* p, T v) {
  static_assert(sizeof(T) == 2 || sizeof(T) == 4 || sizeof(T) == 8, "header words are 2, 4 or 8 bytes");
  if constexpr (sizeof(T) == 8) {
    uint64_t bits;
    std::memcpy(&bits, &v, 8);
    __atomic_store_n(reinterpret_cast<uint64_t*>(p), bits, __ATOMIC_RELAXED);
  } else if constexpr (sizeof(T) == 4) {
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    __atomic_store_n(reinterpret_cast<uint32_t*>(p), bits, __ATOMIC_RELAXED);
  } else {
    uint16_t bits;
    std::memcpy(&bits, &v, 2);
    __atomic_store_n(reinterpret_cast<uint16_t*>(p), bits, __ATOMIC_RELAXED);
  }
}
template <typename T>
inline T same_value_load(const T* p) {
  T v;
  if constexpr (sizeof(T) == 8) {
    const uint64_t bits = __atomic_load_n(reinterpret_cast<const uint64_t*>(p), __ATOMIC_RELAXED);
    std::memcpy(&v, &bits, 8);
  } else if constexpr (sizeof(T) == 4) {
    const uint32_t bits = __atomic_load_n(reinterpret_cast<const uint32_t*>(p), __ATOMIC_RELAXED);
    std::memcpy(&v, &bits, 4);
  } else {
    const uint16_t bits = __atomic_load_n(reinterpret_cast<const uint16_t*>(p), __ATOMIC_RELAXED);
    std::memcpy(&v, &bits, 2);
  }
  return v;
}
}  // namespace bagua

// `__shared__ T name;` of the device build: slot-indexed storage in the block's context.
#define BAGUA_SHARED(T, name, slot) T& name = ::bagua::hostemu::shared_slot<T>(slot)
// `__shared__ T name[count];`
#define BAGUA_SHARED_ARRAY(T, name, count, slot) T* name = ::bagua::hostemu::shared_array<T>((slot), (count))

#else  // device build

#define BAGUA_SHARED(T, name, slot) __shared__ T name
#define BAGUA_SHARED_ARRAY(T, name, count, slot) __shared__ T name[count]

namespace bagua {
// Plain accesses on the device; see the host branch above for why they have a name.
template <typename T>
__device__ __forceinline__ void same_value_store(T* p, T v) {
  *p = v;
}
template <typename T>
__device__ __forceinline__ T same_value_load(const T* p) {
  return *p;
}
}  // namespace bagua

#endif
