// Internal declarations: the CUDA launchers behind kernels.h (defined in the .cu files).
#pragma once

#include "kernels.h"

namespace bagua {
namespace kernels {
namespace cuda {

void divide_inplace(void* x, DType dt, int64_t n, float d, cudaStream_t s);
void add_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s);
void subtract_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s);
void addmul_inplace(void* x, const void* y, float f, DType dt, int64_t n, cudaStream_t s);
void average_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s);
void async_model_average(float* t, const float* r, const float* cp, float nranks, int64_t n, cudaStream_t s);
void copy_bytes(void* dst, const void* src, size_t bytes, cudaStream_t s);
void multi_copy(const MultiCopySeg* segs_dev, int nseg, void* flat, size_t total_bytes, bool gather, cudaStream_t s);
void reduce_chunk_inplace(void* x, DType dt, int64_t chunk, int n_chunks, int target, bool average, cudaStream_t s);
size_t compress_scratch_bytes(int n_chunks, int64_t chunk_size);
void compress_minmax_u8(const void* in, DType dt, int64_t num_real, int64_t chunk, int n_chunks, uint8_t* out,
                        size_t out_bytes, int target, void* scratch, size_t scratch_bytes, cudaStream_t s);
void decompress_minmax_u8(const uint8_t* in, size_t in_bytes, int64_t chunk, int n_chunks, void* out, DType dt,
                          cudaStream_t s);
void sgd_momentum_flat(float* p, const float* g, float* buf, int64_t n, float lr, float momentum, float dampening,
                       float wd, bool nesterov, bool first_step, cudaStream_t s);
void sgd_momentum_flat_shadow(float* p, const float* g, float* buf, void* shadow, int64_t n, float lr, float momentum,
                              float dampening, float wd, bool nesterov, bool first_step, cudaStream_t s);

}  // namespace cuda
}  // namespace kernels
}  // namespace bagua
