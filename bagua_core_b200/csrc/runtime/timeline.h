// Device-side timeline of bucket communication.
//
// When switched on (BAGUA_B200_BUCKET_TIMING=1 or `set_bucket_timing(true)`), every
// communication op brackets the kernels it queues with two timing events on the
// communication stream, and callers may drop named marks on any stream (the trainer marks
// the start of a step and the end of backward on the compute stream).  `collect()` waits for
// the recorded events and returns every span with times in milliseconds relative to the
// first recorded event, which is what it takes to say how long each bucket's kernel ran,
// how far it overlapped the backward pass, and how much communication was left exposed
// after backward had finished.
//
// The reference has no device timing at all: its spans are host times around
// `mark_communication_ready` (bagua-core-internal/src/lib.rs:305-307).
#pragma once

#include <cuda_runtime_api.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "../common.h"

namespace bagua {

struct TimelineSpan {
  std::string name;
  std::string kind;   // "bucket" or "mark"
  double start_ms;    // relative to the first event of the collection
  double end_ms;      // == start_ms for a mark
  uint64_t bytes;     // payload of a bucket span
};

class BucketTimeline {
 public:
  static BucketTimeline& instance();

  void set_enabled(bool on) { enabled_.store(on, std::memory_order_release); }
  bool enabled() const { return enabled_.load(std::memory_order_acquire); }

  // Records the start event on `stream` and returns a ticket for `end` (0 when off or full).
  uint64_t begin(const std::string& name, uint64_t bytes, cudaStream_t stream);
  void end(uint64_t ticket, cudaStream_t stream);
  void mark(const std::string& name, cudaStream_t stream);

  // Synchronises with every recorded event, returns the spans in recording order and
  // forgets them.  Events are recycled.
  std::vector<TimelineSpan> collect();

 private:
  BucketTimeline();
  cudaEvent_t take_event(int device);
  struct Rec {
    std::string name;
    bool is_mark;
    uint64_t bytes;
    cudaEvent_t a, b;
    int device;
    uint64_t id;
    bool closed = false;
  };
  std::atomic<bool> enabled_{false};
  std::mutex mu_;
  std::vector<Rec> recs_;
  uint64_t next_id_ = 1;
  std::vector<std::pair<int, cudaEvent_t>> free_;  // (device, event)
  static constexpr size_t kMaxRecords = 1 << 16;
};

}  // namespace bagua
