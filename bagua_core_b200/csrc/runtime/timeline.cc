#include "timeline.h"

#include <cuda_runtime.h>

namespace bagua {

BucketTimeline::BucketTimeline() { enabled_.store(env_long("BAGUA_B200_BUCKET_TIMING", 0) != 0); }

BucketTimeline& BucketTimeline::instance() {
  static BucketTimeline* t = new BucketTimeline();  // never destroyed: events may outlive the runtime at exit
  return *t;
}

// mu_ held
cudaEvent_t BucketTimeline::take_event(int device) {
  for (size_t i = 0; i < free_.size(); ++i)
    if (free_[i].first == device) {
      cudaEvent_t e = free_[i].second;
      free_[i] = free_.back();
      free_.pop_back();
      return e;
    }
  cudaEvent_t e = nullptr;
  BAGUA_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDefault));
  return e;
}

uint64_t BucketTimeline::begin(const std::string& name, uint64_t bytes, cudaStream_t stream) {
  if (!enabled()) return 0;
  int device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> g(mu_);
  if (recs_.size() >= kMaxRecords) return 0;
  Rec r{name, false, bytes, take_event(device), take_event(device), device, next_id_++};
  BAGUA_CUDA_CHECK(cudaEventRecord(r.a, stream));
  recs_.push_back(std::move(r));
  return recs_.back().id;
}

void BucketTimeline::end(uint64_t ticket, cudaStream_t stream) {
  if (ticket == 0) return;
  std::lock_guard<std::mutex> g(mu_);
  // newest first: the record being closed is almost always the last one.  A collect() between
  // begin and end has taken the record away; then there is nothing to close.
  for (auto it = recs_.rbegin(); it != recs_.rend(); ++it)
    if (it->id == ticket) {
      BAGUA_CUDA_CHECK(cudaEventRecord(it->b, stream));
      it->closed = true;
      return;
    }
}

void BucketTimeline::mark(const std::string& name, cudaStream_t stream) {
  if (!enabled()) return;
  int device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> g(mu_);
  if (recs_.size() >= kMaxRecords) return;
  Rec r{name, true, 0, take_event(device), nullptr, device, next_id_++};
  BAGUA_CUDA_CHECK(cudaEventRecord(r.a, stream));
  recs_.push_back(std::move(r));
}

std::vector<TimelineSpan> BucketTimeline::collect() {
  std::vector<Rec> recs;
  {
    std::lock_guard<std::mutex> g(mu_);
    recs.swap(recs_);
  }
  std::vector<TimelineSpan> out;
  if (recs.empty()) return out;
  out.reserve(recs.size());
  int prev_device = 0;
  cudaGetDevice(&prev_device);
  const Rec& base = recs.front();
  for (const Rec& r : recs) {
    // elapsed time is only defined between events of one device: others are reported against their own first event
    const Rec* origin = &base;
    if (r.device != base.device)
      for (const Rec& q : recs)
        if (q.device == r.device) {
          origin = &q;
          break;
        }
    cudaSetDevice(r.device);
    float a = 0.f, b = 0.f;
    bool ok = cudaEventSynchronize(r.a) == cudaSuccess && cudaEventElapsedTime(&a, origin->a, r.a) == cudaSuccess;
    if (ok && !r.is_mark)
      ok = r.closed && cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&b, origin->a, r.b) == cudaSuccess;
    if (!ok) {
      cudaGetLastError();  // an op that threw between begin and end never recorded its end event
      continue;
    }
    out.push_back(TimelineSpan{r.name, r.is_mark ? "mark" : "bucket", (double)a, r.is_mark ? (double)a : (double)b,
                               r.bytes});
  }
  cudaSetDevice(prev_device);
  {
    std::lock_guard<std::mutex> g(mu_);
    for (const Rec& r : recs) {
      free_.emplace_back(r.device, r.a);
      if (r.b) free_.emplace_back(r.device, r.b);
    }
  }
  return out;
}

}  // namespace bagua
