// Host-side entry points of every tensor kernel, for both device kinds.
//
// Each function takes a `Ctx` naming where the data lives: `device < 0` runs the C++
// restatement on the host (the correctness oracle and the transport-agnostic CPU
// backend), `device >= 0` enqueues the sm_100a kernel on `stream`.  Extents are 64-bit
// (the reference's launchers take `int`, bagua-core-internal/src/kernels/mod.rs:5-136).
//
// Reference parity (bagua-core-internal/kernels/bagua_kernels.cu):
//   divide_inplace 244-255 · add_inplace 220-230 · subtract_inplace 208-218 ·
//   addmul_inplace 232-242 · average_inplace 196-206 · async_model_average 257-266 ·
//   reduce_chunk_inplace 373-400 · array_min_max 312-371 · compress 455-479 ·
//   decompress 481-500.  Half/bf16 inputs are widened to fp32, combined in fp32 and
//   rounded once on store (the reference combines in half precision).
#pragma once

#include <cuda_runtime_api.h>

#include "../common.h"

namespace bagua {
namespace kernels {

struct Ctx {
  int device = -1;            // < 0 → host memory, run on the calling thread
  cudaStream_t stream = 0;    // ignored on the host
  bool is_cuda() const { return device >= 0; }
};

// ---- element-wise -----------------------------------------------------------------
void divide_inplace(void* x, DType dt, int64_t n, float divisor, const Ctx& c);
void add_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c);
void subtract_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c);
void addmul_inplace(void* x, const void* y, float factor, DType dt, int64_t n, const Ctx& c);
void average_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c);
// t[i] += reduced[i] / nranks - copy[i], applied with atomics because the training
// stream may be updating `t` at the same time.  fp32 only.
void async_model_average(float* t, const float* reduced, const float* copy, float nranks, int64_t n,
                         const Ctx& c);
void copy_bytes(void* dst, const void* src, size_t bytes, const Ctx& c);

// Flatten (gather = true: tensors -> flat) or unflatten (flat -> tensors) a list of tensors in
// one launch.  Segments are sorted by `offset` and do not overlap; `segs` is a device array on
// the CUDA path and a host array on the host path.
struct MultiCopySeg {
  void* ptr;                  // the tensor's data
  unsigned long long offset;  // where it sits in the flat buffer, in bytes
  unsigned long long bytes;
};
void multi_copy(const MultiCopySeg* segs, int nseg, void* flat, size_t total_bytes, bool gather, const Ctx& c);

// x viewed as [num_chunks][chunk_size]: column sum (fp32, chunk order 0..n-1), optional
// division by num_chunks, written into chunk `target_chunk`.
void reduce_chunk_inplace(void* x, DType dt, int64_t chunk_size, int num_chunks, int target_chunk,
                          bool average, const Ctx& c);

// ---- MinMaxUInt8 compression --------------------------------------------------------
// Buffer layout (reference: bagua-core-internal/src/datatypes/mod.rs:679-693 and
// bagua_kernels.cu:470,497,537): total = align32(chunk_size*n_chunks) + 32*n_chunks bytes;
// chunk i starts at i*(total/n_chunks): [min:T][max:T][pad to 32 B][chunk_size x u8].
constexpr int kCompressHeaderBytes = 32;
size_t compressed_buffer_size(int n_chunks, int64_t chunk_size, DType dt);

// Scratch needed by the CUDA path of compress (per-block partial min/max); 0 on the host.
size_t compress_scratch_bytes(int n_chunks, int64_t chunk_size);

// Quantise `in` (n_chunks*chunk_size allocated elements, of which `num_real` are real
// data; min/max of a chunk are taken over its real elements only, an all-padding chunk
// gets min=max=0).  target_chunk = -1 → all chunks; otherwise only that chunk is written.
void compress_minmax_u8(const void* in, DType dt, int64_t num_real, int64_t chunk_size, int n_chunks,
                        uint8_t* out, size_t out_bytes, int target_chunk, void* scratch,
                        size_t scratch_bytes, const Ctx& c);
void decompress_minmax_u8(const uint8_t* in, size_t in_bytes, int64_t chunk_size, int n_chunks,
                          void* out, DType dt, const Ctx& c);

// Scalar definition of the quantiser, shared by host code and tests.
struct MinMaxGrid {
  float scale, lower, upper;
};
MinMaxGrid minmax_grid(float mn, float mx);

// ---- fused optimiser steps over flat bucket memory (no reference counterpart) -------
// p -= lr * (momentum buffer update of g (+ weight_decay * p)), torch.optim.SGD semantics.
void sgd_momentum_flat(float* p, const float* g, float* buf, int64_t n, float lr, float momentum,
                       float dampening, float weight_decay, bool nesterov, bool first_step,
                       const Ctx& c);
// The same step, which also writes every updated parameter rounded to bf16 into `shadow`
// (n bf16 values): a model that computes in bf16 then reads its weights from there instead
// of casting the fp32 master copy again in every forward pass.
void sgd_momentum_flat_shadow(float* p, const float* g, float* buf, void* shadow, int64_t n, float lr, float momentum,
                              float dampening, float weight_decay, bool nesterov, bool first_step, const Ctx& c);

}  // namespace kernels
}  // namespace bagua
