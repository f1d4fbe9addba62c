#include "tensor.h"

#include <cuda_runtime.h>

#include "../ops/comm_op.h"

namespace bagua {

std::shared_ptr<PoolRawTensor> PoolRawTensor::allocate(int device, DType dt, int64_t numel, uint64_t stream) {
  auto block = MemoryPool::for_device(device).pull((size_t)numel * dtype_bytes(dt), stream);
  return std::make_shared<PoolRawTensor>(std::move(block), numel, numel, dt, device);
}

namespace tensor_ops {

namespace {
void check_same(const RawTensor& a, const RawTensor& b, const char* what) {
  BAGUA_CHECK(a.dtype() == b.dtype(), Tensor, what << ": dtype mismatch");
  BAGUA_CHECK(a.device_id() == b.device_id(), Tensor, what << ": device mismatch");
  BAGUA_CHECK(a.num_elements_allocated() == b.num_elements_allocated(), Tensor,
              what << ": size mismatch " << a.num_elements_allocated() << " vs " << b.num_elements_allocated());
}
}  // namespace

void clone_from(RawTensor& dst, const RawTensor& src, uint64_t stream) {
  check_same(dst, src, "clone_from");
  kernels::copy_bytes(dst.data_ptr(), src.data_ptr(), dst.bytes_allocated(), dst.ctx(stream));
}
void divide_inplace(RawTensor& t, uint64_t stream, float divisor) {
  kernels::divide_inplace(t.data_ptr(), t.dtype(), t.num_elements_allocated(), divisor, t.ctx(stream));
}
void add_inplace(RawTensor& t, const RawTensor& o, uint64_t stream) {
  check_same(t, o, "add_inplace");
  kernels::add_inplace(t.data_ptr(), o.data_ptr(), t.dtype(), t.num_elements_allocated(), t.ctx(stream));
}
void subtract_inplace(RawTensor& t, const RawTensor& o, uint64_t stream) {
  check_same(t, o, "subtract_inplace");
  kernels::subtract_inplace(t.data_ptr(), o.data_ptr(), t.dtype(), t.num_elements_allocated(), t.ctx(stream));
}
void addmul_inplace(RawTensor& t, const RawTensor& o, float factor, uint64_t stream) {
  check_same(t, o, "addmul_inplace");
  kernels::addmul_inplace(t.data_ptr(), o.data_ptr(), factor, t.dtype(), t.num_elements_allocated(), t.ctx(stream));
}
void average_inplace(RawTensor& t, const RawTensor& o, uint64_t stream) {
  check_same(t, o, "average_inplace");
  kernels::average_inplace(t.data_ptr(), o.data_ptr(), t.dtype(), t.num_elements_allocated(), t.ctx(stream));
}
void async_model_average(RawTensor& t, const RawTensor& reduced, const RawTensor& copy, float nranks,
                         uint64_t stream) {
  check_same(t, reduced, "async_model_average");
  check_same(t, copy, "async_model_average");
  BAGUA_CHECK(t.dtype() == DType::F32, Tensor, "async_model_average supports F32 only");
  kernels::async_model_average((float*)t.data_ptr(), (const float*)reduced.data_ptr(), (const float*)copy.data_ptr(),
                               nranks, t.num_elements_allocated(), t.ctx(stream));
}
static void reduce_chunks(RawTensor& t, int n_chunks, int target, bool avg, uint64_t stream) {
  BAGUA_CHECK(n_chunks > 0 && t.num_elements_allocated() % n_chunks == 0, Tensor,
              "reduce: tensor size " << t.num_elements_allocated() << " is not divisible by " << n_chunks);
  kernels::reduce_chunk_inplace(t.data_ptr(), t.dtype(), t.num_elements_allocated() / n_chunks, n_chunks, target, avg,
                                t.ctx(stream));
}
void reduce_mean_inplace(RawTensor& t, int n_chunks, int target, uint64_t stream) {
  reduce_chunks(t, n_chunks, target, true, stream);
}
void reduce_sum_inplace(RawTensor& t, int n_chunks, int target, uint64_t stream) {
  reduce_chunks(t, n_chunks, target, false, stream);
}

std::shared_ptr<RawTensor> compress(const RawTensor& t, const std::string& method, int n_chunks, uint64_t stream,
                                    int target_chunk) {
  BAGUA_CHECK(method == "MinMaxUInt8", Tensor, "unsupported compression method " << method);
  BAGUA_CHECK(n_chunks > 0 && t.num_elements_allocated() % n_chunks == 0, Tensor,
              "compression tensor size % n_chunks must be 0");
  const int64_t chunk = t.num_elements_allocated() / n_chunks;
  const size_t out_bytes = kernels::compressed_buffer_size(n_chunks, chunk, t.dtype());
  auto out = PoolRawTensor::allocate(t.device_id(), DType::U8, (int64_t)out_bytes, stream);
  std::shared_ptr<PoolBlock> scratch;
  size_t scratch_bytes = 0;
  if (t.device_id() >= 0) {
    scratch_bytes = kernels::compress_scratch_bytes(n_chunks, chunk);
    scratch = MemoryPool::for_device(t.device_id()).pull(scratch_bytes, stream);
  }
  kernels::compress_minmax_u8(t.data_ptr(), t.dtype(), t.num_elements(), chunk, n_chunks, (uint8_t*)out->data_ptr(),
                              out_bytes, target_chunk, scratch ? scratch->ptr() : nullptr, scratch_bytes,
                              t.ctx(stream));
  // The scratch lease returns to the pool here; only a later pull tagged with the same
  // stream can reuse it, and that use is ordered after the kernels above.
  return out;
}

void decompress_from(RawTensor& t, const std::string& method, int n_chunks, const RawTensor& compressed,
                     uint64_t stream) {
  BAGUA_CHECK(method == "MinMaxUInt8", Tensor, "unsupported compression method " << method);
  BAGUA_CHECK(compressed.dtype() == DType::U8, Tensor, "compressed buffer must be U8");
  BAGUA_CHECK(n_chunks > 0 && t.num_elements_allocated() % n_chunks == 0, Tensor,
              "compression tensor size % n_chunks must be 0");
  BAGUA_CHECK(t.device_id() == compressed.device_id(), Tensor, "decompress: device mismatch");
  kernels::decompress_minmax_u8((const uint8_t*)compressed.data_ptr(), (size_t)compressed.num_elements_allocated(),
                                t.num_elements_allocated() / n_chunks, n_chunks, t.data_ptr(), t.dtype(),
                                t.ctx(stream));
}

}  // namespace tensor_ops

// ---------------------------------------------------------------------------------
void BaguaTensor::mark_comm_ready(uint64_t cuda_event) {
  std::unique_lock<std::shared_mutex> g(mu_);
  if (cuda_event == 0) BAGUA_LOG(Debug, "mark comm ready with an event 0, ignoring event");
  ready_ = true;
  ready_event_ = cuda_event;
}
void BaguaTensor::reset_comm_ready() {
  std::unique_lock<std::shared_mutex> g(mu_);
  ready_ = false;
}
bool BaguaTensor::ready_for_comm() const {
  if (is_padding()) return true;
  std::shared_lock<std::shared_mutex> g(mu_);
  return ready_;
}
uint64_t BaguaTensor::take_ready_event() {
  std::unique_lock<std::shared_mutex> g(mu_);
  uint64_t e = ready_event_;
  ready_event_ = 0;
  return e;
}

std::shared_ptr<BaguaTensor> BaguaTensor::compress(const std::string& method, int n_chunks, int target_chunk) const {
  auto r = raw();
  auto out = tensor_ops::compress(*r, method, n_chunks, /*stream=*/0, target_chunk);
  return std::make_shared<BaguaTensor>("compressed_tensor", std::move(out));
}
void BaguaTensor::decompress_from(const std::string& method, int n_chunks, const BaguaTensor& compressed) {
  auto r = raw();
  auto c = compressed.raw();
  tensor_ops::decompress_from(*r, method, n_chunks, *c, /*stream=*/0);
}
void BaguaTensor::copy_to_host(void* dst) const {
  auto r = raw();
  const size_t bytes = (size_t)r->num_elements() * dtype_bytes(r->dtype());
  if (r->device_id() >= 0) {
    BAGUA_CUDA_CHECK(cudaMemcpy(dst, r->data_ptr(), bytes, cudaMemcpyDeviceToHost));
  } else {
    std::memcpy(dst, r->data_ptr(), bytes);
  }
}

// ---------------------------------------------------------------------------------
BaguaBucket::BaguaBucket(std::string name, std::vector<TensorPtr> tensors)
    : name_(std::move(name)), tensors_(std::move(tensors)) {
  BAGUA_CHECK(!tensors_.empty(), Bucket, "bucket must contain at least one tensor");
  dtype_ = tensors_[0]->dtype();
  device_ = tensors_[0]->device_id();
  for (auto& t : tensors_) {
    BAGUA_CHECK(t->dtype() == dtype_, Bucket, "tensors in the same bucket should be of the same dtype");
    BAGUA_CHECK(t->device_id() == device_, Bucket, "tensors in the same bucket should be on the same device");
    BAGUA_CHECK(t->num_elements_allocated() >= t->num_elements(), Bucket,
                "tensors must have allocated at least as many elements as they hold");
  }
}

int64_t BaguaBucket::total_allocated() const {
  int64_t n = 0;
  for (auto& t : tensors_) n += t->num_elements_allocated();
  return n;
}

bool BaguaBucket::contiguous() const {
  const size_t es = dtype_bytes(dtype_);
  uint64_t expect = tensors_[0]->data_ptr();
  for (auto& t : tensors_) {
    if (t->data_ptr() != expect) return false;
    expect += (uint64_t)t->num_elements_allocated() * es;
  }
  return true;
}

bool BaguaBucket::ready_for_comm() const {
  // Asked after every tensor that becomes ready.  A trainer lists a bucket's tensors in the order
  // their gradients appear, so the ones at the back are the last to become ready: looking from the
  // back meets an unready tensor at once, where looking from the front walks over all that are
  // ready already (one lock each) before it finds one.
  for (auto it = tensors_.rbegin(); it != tensors_.rend(); ++it)
    if (!(*it)->ready_for_comm()) return false;
  return true;
}
void BaguaBucket::reset_comm_ready() {
  for (auto& t : tensors_) t->reset_comm_ready();
}
bool BaguaBucket::all_padding() const {
  for (auto& t : tensors_)
    if (!t->is_padding()) return false;
  return true;
}

void BaguaBucket::append_op(std::shared_ptr<CommOp> op) {
  std::lock_guard<std::mutex> g(mu_);
  ops_.push_back(std::move(op));
}
void BaguaBucket::clear_ops() {
  std::lock_guard<std::mutex> g(mu_);
  ops_.clear();
}
std::vector<std::shared_ptr<CommOp>> BaguaBucket::ops_snapshot() const {
  std::lock_guard<std::mutex> g(mu_);
  return ops_;
}
std::string BaguaBucket::describe_ops() const {
  std::lock_guard<std::mutex> g(mu_);
  std::ostringstream oss;
  oss << "[";
  for (size_t i = 0; i < ops_.size(); ++i) oss << (i ? ", " : "") << ops_[i]->describe();
  oss << "]";
  return oss.str();
}

CommunicationTensor BaguaBucket::get_communication_tensor(uint64_t stream, bool force_copy,
                                                          bool force_not_copy_back) {
  CommunicationTensor ct;
  ct.stream = stream;
  ct.bucket_tensors = tensors_;
  for (auto& t : tensors_) {
    uint64_t ev = t->take_ready_event();
    if (ev != 0 && device_ >= 0)
      BAGUA_CUDA_CHECK(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0));
  }
  const int64_t total = total_allocated();
  if (!force_copy && contiguous()) {
    int64_t real = 0;
    for (auto& t : tensors_) real += t->num_elements_allocated();
    ct.raw = std::make_shared<PoolRawTensor>((void*)(uintptr_t)tensors_[0]->data_ptr(), nullptr, real, total, dtype_,
                                             device_);
    ct.need_copy_back = false;
    return ct;
  }
  // Staged: one launch gathers every tensor into a pool buffer (the reference issues one copy
  // per tensor, datatypes/mod.rs:1012-1023).
  auto buf = PoolRawTensor::allocate(device_, dtype_, total, stream);
  const size_t es = dtype_bytes(dtype_);
  unsigned long long off = 0;
  kernels::Ctx c{device_, (cudaStream_t)stream};
  ct.segments.reserve(tensors_.size());
  for (auto& t : tensors_) {
    const unsigned long long bytes = (unsigned long long)t->num_elements_allocated() * es;
    if (bytes) ct.segments.push_back(kernels::MultiCopySeg{(void*)(uintptr_t)t->data_ptr(), off, bytes});
    off += bytes;
  }
  const kernels::MultiCopySeg* table = ct.segments.data();
  if (device_ >= 0 && !ct.segments.empty()) {
    const size_t tbytes = ct.segments.size() * sizeof(kernels::MultiCopySeg);
    const bool same = seg_cache_dev_ && seg_cache_.size() == ct.segments.size() &&
                      std::memcmp(seg_cache_.data(), ct.segments.data(), tbytes) == 0;
    if (!same) {
      // the stream orders the upload before the kernels that read it and after those that read the old
      // table; the source is pageable memory, which the runtime stages before the call returns
      seg_cache_dev_ = PoolRawTensor::allocate(device_, DType::U8, (int64_t)tbytes, stream);
      seg_cache_ = ct.segments;
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(seg_cache_dev_->data_ptr(), seg_cache_.data(), tbytes, cudaMemcpyHostToDevice,
                                       (cudaStream_t)stream));
    }
    ct.segments_dev = seg_cache_dev_;
    table = (const kernels::MultiCopySeg*)seg_cache_dev_->data_ptr();
  }
  kernels::multi_copy(table, (int)ct.segments.size(), buf->data_ptr(), (size_t)off, /*gather=*/true, c);
  ct.raw = buf;
  ct.staged = true;
  ct.need_copy_back = !force_not_copy_back;
  return ct;
}

void CommunicationTensor::finish(bool sync_stream) {
  if (!raw) return;
  const int device = raw->device_id();
  if (need_copy_back && !segments.empty()) {
    // one launch scatters the result back (reference: one copy per tensor, datatypes/mod.rs:1048-1059)
    kernels::Ctx c{device, (cudaStream_t)stream};
    const kernels::MultiCopySeg* table =
        segments_dev ? (const kernels::MultiCopySeg*)segments_dev->data_ptr() : segments.data();
    kernels::multi_copy(table, (int)segments.size(), raw->data_ptr(), raw->bytes_allocated(), /*gather=*/false, c);
  }
  // Pool leases are recycled per stream, so no host synchronisation is needed for
  // correctness; it happens only in reference-faithful mode.
  if (device >= 0 && sync_stream)
    BAGUA_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  raw.reset();
}

}  // namespace bagua
