// Tensor and bucket abstractions of the communication engine.
//
// `RawTensor` is a view {data_ptr, numel, numel_allocated, dtype, device}.  Two
// implementations: a framework tensor (an `at::Tensor` held by the bindings, queried
// through its public C++ API — the reference reads private libtorch struct offsets,
// bagua-core-internal/src/datatypes/mod.rs:525-641) and a pool-owned buffer
// (`PoolRawTensor`, reference `BaguaTensorRaw`, datatypes/mod.rs:78-86,643-663).
//
// `BaguaTensor` adds the name and the readiness state the scheduler tracks
// (datatypes/mod.rs:751-910); `BaguaBucket` is a named list of same-dtype, same-device
// tensors with an ordered list of communication ops (datatypes/mod.rs:1072-1267).
#pragma once

#include <functional>
#include <shared_mutex>

#include "../common.h"
#include "../kernels/kernels.h"
#include "../pool/resource_pool.h"

namespace bagua {

class CommOp;
class SingleCommunicator;

class RawTensor {
 public:
  virtual ~RawTensor() = default;
  virtual void* data_ptr() const = 0;
  virtual int64_t num_elements() const = 0;
  virtual int64_t num_elements_allocated() const = 0;
  virtual int device_id() const = 0;  // -1 → host memory
  virtual DType dtype() const = 0;
  size_t bytes_allocated() const { return (size_t)num_elements_allocated() * dtype_bytes(dtype()); }
  kernels::Ctx ctx(uint64_t stream) const { return kernels::Ctx{device_id(), (cudaStream_t)stream}; }
};

class PoolRawTensor : public RawTensor {
 public:
  PoolRawTensor(std::shared_ptr<PoolBlock> block, int64_t numel, int64_t numel_alloc, DType dt, int device)
      : block_(std::move(block)), ptr_(block_->ptr()), numel_(numel), alloc_(numel_alloc), dt_(dt), device_(device) {}
  // a view into memory someone else keeps alive (`keep` may be null for caller-owned memory)
  PoolRawTensor(void* ptr, std::shared_ptr<void> keep, int64_t numel, int64_t numel_alloc, DType dt, int device)
      : keep_(std::move(keep)), ptr_(ptr), numel_(numel), alloc_(numel_alloc), dt_(dt), device_(device) {}
  void* data_ptr() const override { return ptr_; }
  int64_t num_elements() const override { return numel_; }
  int64_t num_elements_allocated() const override { return alloc_; }
  int device_id() const override { return device_; }
  DType dtype() const override { return dt_; }

  static std::shared_ptr<PoolRawTensor> allocate(int device, DType dt, int64_t numel, uint64_t stream = 0);

 private:
  std::shared_ptr<PoolBlock> block_;
  std::shared_ptr<void> keep_;
  void* ptr_;
  int64_t numel_, alloc_;
  DType dt_;
  int device_;
};

// ---- tensor math on raw views (reference trait RawBaguaTensor, datatypes/mod.rs:88-523)
namespace tensor_ops {
void clone_from(RawTensor& dst, const RawTensor& src, uint64_t stream);
void divide_inplace(RawTensor& t, uint64_t stream, float divisor);
void add_inplace(RawTensor& t, const RawTensor& o, uint64_t stream);
void subtract_inplace(RawTensor& t, const RawTensor& o, uint64_t stream);
void addmul_inplace(RawTensor& t, const RawTensor& o, float factor, uint64_t stream);
void average_inplace(RawTensor& t, const RawTensor& o, uint64_t stream);
void async_model_average(RawTensor& t, const RawTensor& reduced, const RawTensor& copy, float nranks, uint64_t stream);
void reduce_mean_inplace(RawTensor& t, int n_chunks, int target_chunk, uint64_t stream);
void reduce_sum_inplace(RawTensor& t, int n_chunks, int target_chunk, uint64_t stream);
// "MinMaxUInt8" is the only method.  Returns a pool-owned U8 tensor.
std::shared_ptr<RawTensor> compress(const RawTensor& t, const std::string& method, int n_chunks, uint64_t stream,
                                    int target_chunk);
void decompress_from(RawTensor& t, const std::string& method, int n_chunks, const RawTensor& compressed,
                     uint64_t stream);
}  // namespace tensor_ops

class BaguaTensor {
 public:
  BaguaTensor(std::string name, std::shared_ptr<RawTensor> raw) : name_(std::move(name)), raw_(std::move(raw)) {}

  const std::string& name() const { return name_; }
  std::shared_ptr<RawTensor> raw() const {
    std::shared_lock<std::shared_mutex> g(mu_);
    return raw_;
  }
  // event == 0 means "ready, nothing to wait for on the stream"
  void mark_comm_ready(uint64_t cuda_event);
  void reset_comm_ready();
  // padding tensors (name prefix "bagua_padding_tensor") are always ready
  bool ready_for_comm() const;
  bool is_padding() const { return name_.rfind("bagua_padding_tensor", 0) == 0; }
  // Returns the stored ready event and clears it.
  uint64_t take_ready_event();

  uint64_t data_ptr() const { return (uint64_t)(uintptr_t)raw()->data_ptr(); }
  int device_id() const { return raw()->device_id(); }
  int64_t num_elements() const { return raw()->num_elements(); }
  int64_t num_elements_allocated() const { return raw()->num_elements_allocated(); }
  DType dtype() const { return raw()->dtype(); }

  // Run on the legacy default stream, like the reference (datatypes/mod.rs:829,882).
  std::shared_ptr<BaguaTensor> compress(const std::string& method, int n_chunks, int target_chunk) const;
  void decompress_from(const std::string& method, int n_chunks, const BaguaTensor& compressed);
  // Synchronous copy to host memory (bytes = numel * dtype size).
  void copy_to_host(void* dst) const;

 private:
  const std::string name_;
  mutable std::shared_mutex mu_;
  std::shared_ptr<RawTensor> raw_;
  bool ready_ = false;
  uint64_t ready_event_ = 0;
};

using TensorPtr = std::shared_ptr<BaguaTensor>;

// The flat view an op communicates on: either an alias of the bucket's tensors (when
// they are laid out back to back) or a staged copy taken from the pool.  `finish()`
// copies a staged buffer back and, in reference-faithful mode, synchronises the stream.
class CommunicationTensor {
 public:
  std::shared_ptr<RawTensor> raw;
  bool need_copy_back = false;
  bool staged = false;  // `raw` is a pool buffer holding a copy of the bucket
  uint64_t stream = 0;
  std::vector<TensorPtr> bucket_tensors;
  // staged: where every tensor sits in `raw`; on a GPU the same table also lives on the device
  std::vector<kernels::MultiCopySeg> segments;
  std::shared_ptr<RawTensor> segments_dev;
  void finish(bool sync_stream);
};

class BaguaBucket {
 public:
  // Validation: non-empty, same dtype, same device, allocated >= numel.
  BaguaBucket(std::string name, std::vector<TensorPtr> tensors);

  const std::string& name() const { return name_; }
  const std::vector<TensorPtr>& tensors() const { return tensors_; }
  DType dtype() const { return dtype_; }
  int device_id() const { return device_; }
  int64_t total_allocated() const;
  bool contiguous() const;  // tensors address-adjacent in list order

  bool ready_for_comm() const;
  void reset_comm_ready();
  bool all_padding() const;

  void append_op(std::shared_ptr<CommOp> op);
  void clear_ops();
  std::vector<std::shared_ptr<CommOp>> ops_snapshot() const;
  std::string describe_ops() const;

  // Waits (stream-side) on every tensor's ready event, then aliases or stages.
  CommunicationTensor get_communication_tensor(uint64_t stream, bool force_copy, bool force_not_copy_back);

  std::mutex& exec_mutex() { return exec_mu_; }

 private:
  const std::string name_;
  std::vector<TensorPtr> tensors_;
  DType dtype_;
  int device_;
  mutable std::mutex mu_;       // guards ops_
  std::mutex exec_mu_;          // serialises op execution on this bucket
  std::vector<std::shared_ptr<CommOp>> ops_;
  // Device copy of the flatten table, re-uploaded only when a tensor has moved (exec_mu_ held).
  std::vector<kernels::MultiCopySeg> seg_cache_;
  std::shared_ptr<RawTensor> seg_cache_dev_;
};

using BucketPtr = std::shared_ptr<BaguaBucket>;

}  // namespace bagua
