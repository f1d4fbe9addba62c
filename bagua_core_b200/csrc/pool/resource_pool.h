// Caching pools for device (or host) scratch memory and CUDA events.
//
// Memory: one pool per device, size classes are powers of two starting at 2 KiB; a freed
// block returns to its class's free list instead of `cudaFree` (allocation on the
// communication path must never synchronise the device).  Device index -1 is host
// memory for the CPU backend.  Events: created with cudaEventDisableTiming and recycled.
// With guards on (BAGUA_B200_POOL_GUARD=1 or set_guard(true)) every new block gets 256 bytes
// of a fixed pattern in front of it and behind its capacity; check_guards() reports blocks
// whose pattern was overwritten: a check that needs no external memory-checking tool and finds
// an out-of-range store of a kernel into pool memory after a test.
// A lease owns its resource until destroyed — the reference copies the raw event out of
// a pool guard that is dropped at once (bagua-core-internal/src/comm_ops/
// decentralized_full_precision_asynchronous.rs:78,107), which this design rules out.
//
// Reference: bagua-core-internal/src/resource_pool/mod.rs:4-98.
#pragma once

#include <cuda_runtime_api.h>

#include <array>
#include <map>
#include <set>

#include "../common.h"

namespace bagua {

class MemoryPool;

// RAII lease of a pooled block.
class PoolBlock {
 public:
  PoolBlock(MemoryPool* pool, void* ptr, size_t bytes, size_t cls, uint64_t tag)
      : pool_(pool), ptr_(ptr), bytes_(bytes), cls_(cls), tag_(tag) {}
  ~PoolBlock();
  PoolBlock(const PoolBlock&) = delete;
  PoolBlock& operator=(const PoolBlock&) = delete;
  void* ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }       // requested size
  size_t capacity() const { return cls_; }      // size-class capacity

 private:
  MemoryPool* pool_;
  void* ptr_;
  size_t bytes_, cls_;
  uint64_t tag_;
};

struct PoolStats {
  uint64_t device_allocs = 0;   // calls that reached cudaMalloc / malloc
  uint64_t pulls = 0;           // leases handed out
  uint64_t bytes_reserved = 0;  // currently held from the device
  uint64_t bytes_in_use = 0;
  uint64_t guard_violations = 0;  // blocks found with an overwritten guard region so far
};

class MemoryPool {
 public:
  static constexpr size_t kMinClass = 2048;
  static constexpr int kMaxDevices = 64;

  explicit MemoryPool(int device) : device_(device) {}
  ~MemoryPool();

  // Throws BaguaError(MemPool) when the device allocation fails.  `stream_tag` is the
  // stream the block will be used on: a freed block is only handed to a later pull with
  // the same tag, so reuse is always ordered by that stream (no host synchronisation
  // is needed before a lease is dropped).
  std::shared_ptr<PoolBlock> pull(size_t bytes, uint64_t stream_tag = 0);
  void release_cached();  // returns free blocks to the device
  PoolStats stats() const;
  int device() const { return device_; }

  static size_t size_class(size_t bytes);
  // device in [-1, kMaxDevices)
  static MemoryPool& for_device(int device);

  // Guard regions around blocks allocated from now on (all pools).
  static constexpr size_t kGuardBytes = 256;
  static constexpr unsigned char kGuardPattern = 0xC5;
  static void set_guard(bool on);
  static bool guard();
  // Checks the guard regions of every guarded block, leased or cached, and returns how many
  // are damaged (each is logged once with the offset of its first damaged byte and counted in
  // stats().guard_violations).  For a device pool this synchronises the device: call it
  // between steps, not while a stream is being captured.
  size_t check_guards();

 private:
  friend class PoolBlock;
  void give_back(void* ptr, size_t cls, uint64_t tag);

  const int device_;
  mutable std::mutex mu_;
  std::map<std::pair<size_t, uint64_t>, std::vector<void*>> free_;
  std::map<void*, size_t> guarded_;  // block -> capacity, for blocks that have guard regions
  std::set<void*> reported_;         // guarded blocks already reported as damaged
  PoolStats stats_;
};

class EventPool;
class EventLease {
 public:
  EventLease(EventPool* pool, cudaEvent_t ev) : pool_(pool), ev_(ev) {}
  ~EventLease();
  EventLease(const EventLease&) = delete;
  EventLease& operator=(const EventLease&) = delete;
  cudaEvent_t get() const { return ev_; }

 private:
  EventPool* pool_;
  cudaEvent_t ev_;
};

class EventPool {
 public:
  ~EventPool();
  // The calling thread's current device owns the event.
  std::unique_ptr<EventLease> take();
  size_t cached() const;
  static EventPool& instance();

 private:
  friend class EventLease;
  void give_back(cudaEvent_t ev);
  mutable std::mutex mu_;
  std::map<int, std::vector<cudaEvent_t>> free_;  // per device
  std::map<cudaEvent_t, int> owner_;
};

}  // namespace bagua
