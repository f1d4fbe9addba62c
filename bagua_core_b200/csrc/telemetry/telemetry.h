// Span telemetry for the autotune service.
//
// Reference: bagua-opentelemetry (src/lib.rs:8-21, src/exporter/mod.rs:14-62,
// src/exporter/agent.rs:3-44).  When AUTO_TUNE_SERVER_ADDR is set, every
// `mark_communication_ready` produces a `tensor_ready` span; spans are batched and
// POSTed as {"spans":[{trace_id, action, tensor_name, start_time, end_time}]} (times in
// ms since the epoch) to http://<addr>/api/v1/report_tensor_execution_order.  Export
// failures are warnings only.  Besides `tensor_ready`, this engine emits
// `bucket_scheduled` and `bucket_executed` spans (tensor_name = bucket name).
//
// Implementation: a mutex-protected queue and one flusher thread with a minimal
// HTTP/1.1 client on a blocking socket; nothing on the hot path but a queue push.
#pragma once

#include <condition_variable>
#include <deque>
#include <thread>

#include "../common.h"

namespace bagua {

struct Span {
  unsigned __int128 trace_id;
  std::string action;
  std::string tensor_name;
  uint64_t start_ms, end_ms;
};

class Telemetry {
 public:
  static Telemetry& instance();
  // Idempotent.  `addr` = "host:port".
  void init(const std::string& addr);
  // Reads AUTO_TUNE_SERVER_ADDR once per process.
  void init_from_env_once();
  bool enabled() const { return enabled_.load(std::memory_order_acquire); }
  void record(const std::string& action, const std::string& tensor_name, uint64_t start_ms, uint64_t end_ms);
  // Blocks until the queue is drained (or `timeout_ms` elapsed).  Returns spans exported so far.
  uint64_t flush(int timeout_ms = 2000);
  void shutdown();
  uint64_t exported() const { return exported_.load(); }
  uint64_t failed_batches() const { return failed_.load(); }

  static std::string to_json(const std::vector<Span>& batch);

 private:
  Telemetry() = default;
  ~Telemetry();
  void run();
  bool post(const std::string& body);

  std::atomic<bool> enabled_{false};
  std::string host_;
  int port_ = 80;
  std::mutex mu_;
  std::condition_variable cv_, drained_;
  std::deque<Span> queue_;
  bool stop_ = false, busy_ = false;
  std::thread thread_;
  std::atomic<uint64_t> exported_{0}, failed_{0};
  std::once_flag env_once_;
};

}  // namespace bagua
