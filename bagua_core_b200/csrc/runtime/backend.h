// The communication backend: ordered-bucket scheduler, worker thread and watchdog.
//
// Reference: BaguaCommBackend (bagua-core-internal/src/lib.rs:125-337).
//   * `register_ordered_buckets` fixes the order in which buckets are communicated.
//   * `mark_communication_ready(tensor, event)` marks a tensor; while the FRONT bucket
//     of the queue is fully ready it is rotated to the back and scheduled.  Only the
//     front is ever tested, so every rank issues buckets in the registered order no
//     matter in which order gradients arrive.
//   * scheduling = pushing {bucket, snapshot of its ops, completion event} into a
//     bounded channel (back-pressure) consumed by ONE worker thread, which runs the ops.
//   * `wait_pending_comm_ops` blocks until every scheduled bucket has been executed by
//     the worker and returns how many there were.
//   * a watchdog thread reports a bucket whose ops do not finish within the timeout
//     (reference: 300 s, then panic).  Here the timeout is configurable and the failure
//     is delivered as an exception from `wait_pending_comm_ops` rather than by exiting.
//
// Differences on purpose: a bucket whose tensors are all padding is rejected at
// registration (the reference would spin forever on it); op errors are caught on the
// worker and re-raised to the caller of `wait_pending_comm_ops`.
#pragma once

#include <deque>
#include <thread>
#include <unordered_map>
#include <unordered_set>

#include "../ops/comm_op.h"
#include "../tensor/tensor.h"
#include "channel.h"

namespace bagua {

struct ScheduledCommOp {
  std::string name;
  BucketPtr bucket;
  std::vector<std::shared_ptr<CommOp>> ops;
  EventChannel event{"comm_op"};
};

class CommBackend {
 public:
  // device_id < 0: host-only backend (no CUDA calls).
  CommBackend(size_t schedule_channel_cap, int device_id);
  ~CommBackend();
  CommBackend(const CommBackend&) = delete;

  void register_ordered_buckets(const std::vector<BucketPtr>& buckets);
  void mark_communication_ready(const TensorPtr& tensor, uint64_t ready_cuda_event);
  size_t wait_pending_comm_ops();

  // seconds; <= 0 disables the watchdog.  Default: BAGUA_B200_WATCHDOG_S or 300.
  void set_watchdog_timeout(double seconds) { watchdog_s_.store(seconds); }
  double watchdog_timeout() const { return watchdog_s_.load(); }
  int device_id() const { return device_id_; }
  size_t pending() const { return not_waited_.size(); }

 private:
  bool should_schedule() const;
  void schedule_comm(const BucketPtr& bucket);
  void worker_loop();
  void monitor_loop();

  const int device_id_;
  std::deque<BucketPtr> ordered_buckets_;
  std::mutex mu_;  // guards ordered_buckets_ and registration state

  Channel<std::shared_ptr<ScheduledCommOp>> schedule_;
  Channel<EventChannel> not_waited_;
  struct MonitorMsg {
    std::string bucket;
    EventChannel done{"monitor"};
  };
  Channel<std::shared_ptr<MonitorMsg>> monitor_;
  std::atomic<double> watchdog_s_;
  std::mutex err_mu_;
  std::string watchdog_error_;
  std::thread worker_, monitor_thread_;
};

}  // namespace bagua
