#include "backend.h"

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include "../telemetry/telemetry.h"

namespace bagua {

CommBackend::CommBackend(size_t cap, int device_id)
    : device_id_(device_id), schedule_(cap == 0 ? 1 : cap), not_waited_(0), monitor_(0),
      watchdog_s_(env_double("BAGUA_B200_WATCHDOG_S", 300.0)) {
  if (device_id_ >= 0) BAGUA_CUDA_CHECK(cudaSetDevice(device_id_));
  Telemetry::instance().init_from_env_once();
  worker_ = std::thread([this] { worker_loop(); });
  monitor_thread_ = std::thread([this] { monitor_loop(); });
}

CommBackend::~CommBackend() {
  schedule_.close();
  monitor_.close();
  if (worker_.joinable()) worker_.join();
  if (monitor_thread_.joinable()) monitor_thread_.join();
}

void CommBackend::worker_loop() {
  if (device_id_ >= 0) {
    cudaError_t e = cudaSetDevice(device_id_);
    if (e != cudaSuccess) BAGUA_LOG(Error, "comm worker cannot select device " << device_id_);
  }
  for (;;) {
    auto item = schedule_.recv();
    if (!item) return;
    auto& op = **item;
    BAGUA_LOG(Debug, "worker received scheduled communication operation " << op.name);
    auto mon = std::make_shared<MonitorMsg>();
    mon->bucket = op.bucket->name();
    monitor_.send(mon);
    if (log_enabled(LogLevel::Debug)) {
      std::string names;
      for (auto& t : op.bucket->tensors()) names += (names.empty() ? "" : ",") + t->name();
      BAGUA_LOG(Debug, "executing communication op `" << op.name << "` on bucket `" << op.bucket->name()
                                                      << "`, tensors [" << names << "]");
    }
    const uint64_t t0 = now_ms();
    std::string err;
    // Optional NVTX range per bucket (BAGUA_B200_NVTX=1) so that profiler timelines line up
    // with bucket names; a no-op when no tool is attached.
    static const bool nvtx = env_long("BAGUA_B200_NVTX", 0) != 0;
    if (nvtx) nvtxRangePushA(op.bucket->name().c_str());
    try {
      for (auto& o : op.ops) {
        o->execute_background_communication(op.bucket);
        EngineStats::global().ops_executed++;
      }
    } catch (const std::exception& e) {
      err = e.what();
      BAGUA_LOG(Error, "communication op on bucket `" << op.bucket->name() << "` failed: " << err);
    }
    if (nvtx) nvtxRangePop();
    Telemetry::instance().record("bucket_executed", op.bucket->name(), t0, now_ms());
    if (err.empty())
      op.event.finish();
    else
      op.event.fail(err);
    mon->done.finish();
    BAGUA_LOG(Debug, "comm op executed: " << op.name);
  }
}

void CommBackend::monitor_loop() {
  for (;;) {
    auto msg = monitor_.recv();
    if (!msg) return;
    for (;;) {
      const double limit = watchdog_s_.load();
      if (limit <= 0) {
        (*msg)->done.wait();
        break;
      }
      if ((*msg)->done.wait_for(std::chrono::milliseconds((int64_t)(limit * 1000)))) break;
      const std::string what =
          "bucket `" + (*msg)->bucket + "` comm op has not finished for " + fmt_double(limit) + " s";
      BAGUA_LOG(Error, what);
      {
        std::lock_guard<std::mutex> g(err_mu_);
        if (watchdog_error_.empty()) watchdog_error_ = what;
      }
      // keep waiting: the op may still complete; the error is reported to the next waiter
      (*msg)->done.wait();
      break;
    }
  }
}

void CommBackend::register_ordered_buckets(const std::vector<BucketPtr>& buckets) {
  wait_pending_comm_ops();
  std::lock_guard<std::mutex> g(mu_);
  ordered_buckets_.clear();
  std::unordered_set<std::string> names;
  std::unordered_set<uint64_t> ptrs;
  for (auto& b : buckets) {
    BAGUA_CHECK(!b->all_padding(), Bucket,
                "bucket `" << b->name() << "` contains only padding tensors and would always be ready");
    for (auto& t : b->tensors()) {
      const uint64_t p = t->data_ptr();
      if (names.count(t->name()) || ptrs.count(p)) {
        ordered_buckets_.clear();
        throw BaguaError(ErrorKind::Tensor,
                         "duplicated tensor detected, name " + t->name() + ", ptr " + std::to_string(p));
      }
      names.insert(t->name());
      ptrs.insert(p);
    }
    ordered_buckets_.push_back(b);
  }
}

bool CommBackend::should_schedule() const {
  if (ordered_buckets_.empty()) throw BaguaError(ErrorKind::Backend, "ordered buckets not yet set in comm backend");
  return ordered_buckets_.front()->ready_for_comm();
}

void CommBackend::schedule_comm(const BucketPtr& bucket) {
  auto op = std::make_shared<ScheduledCommOp>();
  op->name = "comm op for bucket " + bucket->name();
  op->bucket = bucket;
  op->ops = bucket->ops_snapshot();
  EventChannel ev = op->event;
  const uint64_t t0 = now_ms();
  if (!schedule_.send(std::move(op))) throw BaguaError(ErrorKind::InternalChannel, "schedule channel is closed");
  not_waited_.send(ev);
  EngineStats::global().buckets_scheduled++;
  Telemetry::instance().record("bucket_scheduled", bucket->name(), t0, now_ms());
}

void CommBackend::mark_communication_ready(const TensorPtr& tensor, uint64_t ready_cuda_event) {
  const uint64_t t0 = now_ms();
  tensor->mark_comm_ready(ready_cuda_event);
  {
    std::lock_guard<std::mutex> g(mu_);
    while (should_schedule()) {
      BucketPtr bucket = ordered_buckets_.front();
      ordered_buckets_.pop_front();
      BAGUA_LOG(Debug, "bucket " << bucket->name() << " ready for communication");
      bucket->reset_comm_ready();
      ordered_buckets_.push_back(bucket);
      schedule_comm(bucket);
    }
  }
  Telemetry::instance().record("tensor_ready", tensor->name(), t0, now_ms());
}

size_t CommBackend::wait_pending_comm_ops() {
  size_t n = 0;
  std::string first_error;
  for (;;) {
    auto ev = not_waited_.try_recv();
    if (!ev) break;
    // Poll so that a watchdog report reaches the caller even if the op never returns.
    while (!ev->wait_for(std::chrono::milliseconds(200))) {
      std::lock_guard<std::mutex> g(err_mu_);
      if (!watchdog_error_.empty()) {
        std::string w = watchdog_error_;
        watchdog_error_.clear();
        // the op is still running: a later wait must still see how it ended
        not_waited_.send(*ev);
        throw BaguaError(ErrorKind::Backend, "watchdog: " + w);
      }
    }
    std::string err = ev->wait();
    if (!err.empty() && first_error.empty()) first_error = err;
    ++n;
  }
  {
    std::lock_guard<std::mutex> g(err_mu_);
    if (first_error.empty() && !watchdog_error_.empty()) first_error = "watchdog: " + watchdog_error_;
    watchdog_error_.clear();
  }
  if (!first_error.empty()) throw BaguaError(ErrorKind::Backend, "communication failed: " + first_error);
  // Every bucket has been queued; kernels of earlier buckets (or steps) may have given up on a
  // peer in the meantime.  Their status records are host-mapped, so looking costs a few loads.
  if (device_id_ >= 0) SingleCommunicator::check_all_device_status();
  return n;
}

}  // namespace bagua
