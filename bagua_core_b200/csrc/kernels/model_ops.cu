// Fused bias + ReLU (forward, in place) and its backward with the bias-gradient reduction,
// on channels-last bf16 activations viewed as [rows, C]; see model_ops.h.
//
// Both kernels are pure streams over the activation: 16-byte vectors (8 channels), every
// warp reads whole contiguous rows, grids are a small multiple of the 148 SMs and loop with a
// grid stride.  The backward keeps one fp32 accumulator per channel of the thread's vector
// across all rows it visits, folds the block's accumulators through shared memory and writes
// one partial row per block; a second tiny kernel adds the partial rows in block order, so the
// bias gradient is bit-reproducible.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common.h"
#include "model_ops.h"
#include "model_ops_bodies.cuh"

namespace bagua {
namespace model_ops {

namespace {

using namespace bodies;

__global__ void __launch_bounds__(kThreads)
    bias_relu_kernel(uint4* __restrict__ z, const __nv_bfloat16* __restrict__ bias, int64_t nvec, int cgroups) {
  bias_relu_body(z, bias, nvec, cgroups);
}
__global__ void __launch_bounds__(kThreads)
    bias_relu_backward_kernel(const uint4* dy, const uint4* __restrict__ y, uint4* dz, float* __restrict__ partial,
                              int64_t rows, int cgroups) {
  __shared__ float s_acc[kThreads * 8];
  bias_relu_backward_body(dy, y, dz, partial, rows, cgroups, s_acc);
}
__global__ void bias_grad_finish_kernel(const float* __restrict__ partial, float* __restrict__ db, int blocks, int C) {
  bias_grad_finish_body(partial, db, blocks, C);
}
__global__ void __launch_bounds__(kThreads)
    maxpool2x2_forward_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t nvec_out, int64_t Wo,
                              int64_t W, int cgroups) {
  maxpool2x2_forward_body(x, y, nvec_out, Wo, W, cgroups);
}
__global__ void __launch_bounds__(kThreads)
    maxpool2x2_backward_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, uint4* __restrict__ dx,
                               int64_t nvec_out, int64_t Wo, int64_t W, int cgroups) {
  maxpool2x2_backward_body(x, dy, dx, nvec_out, Wo, W, cgroups);
}

__global__ void __launch_bounds__(kThreads)
    bias_relu_pool_kernel(uint4* __restrict__ y, uint4* __restrict__ p, const __nv_bfloat16* __restrict__ bias,
                          int64_t pooled_pixels, int64_t Wo, int64_t W, int cgroups) {
  bias_relu_pool_body(y, p, bias, pooled_pixels, Wo, W, cgroups);
}
__global__ void __launch_bounds__(kThreads)
    bias_relu_pool_backward_kernel(const uint4* __restrict__ dp, const uint4* __restrict__ y, uint4* __restrict__ dz,
                                   float* __restrict__ partial, int64_t pooled_rows, int64_t Wo, int64_t W, int cgroups) {
  __shared__ float s_acc[kThreads * 8];
  bias_relu_pool_backward_body(dp, y, dz, partial, pooled_rows, Wo, W, cgroups, s_acc);
}

int pool_grid(int64_t nvec_out) {
  const int64_t want = (nvec_out + kThreads - 1) / kThreads;
  return (int)std::max<int64_t>(1, std::min<int64_t>(want, 148 * 8));
}

int backward_blocks(int64_t rows, int C) {
  const int rows_per_iter = kThreads / (C / 8);
  const int64_t want = (rows + rows_per_iter - 1) / rows_per_iter;
  return (int)std::max<int64_t>(1, std::min<int64_t>(want, kMaxBlocks));
}

}  // namespace

static_assert(kThreads == kBlockThreads, "bias_relu_supported() assumes the kernels' block size");

void bias_relu_inplace_bf16(void* z, const void* bias, int64_t rows, int C, cudaStream_t stream) {
  BAGUA_CHECK(bias_relu_supported(rows, C) && (uintptr_t)z % 16 == 0, Tensor,
              "fused bias+ReLU: unsupported shape [" << rows << ", " << C << "] or unaligned activation");
  const int64_t nvec = rows * (C / 8);
  const int64_t want = (nvec + (int64_t)kThreads * 4 - 1) / ((int64_t)kThreads * 4);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(want, 148 * 8));
  bias_relu_kernel<<<grid, kThreads, 0, stream>>>((uint4*)z, (const __nv_bfloat16*)bias, nvec, C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

size_t bias_relu_backward_scratch_bytes(int64_t rows, int C) {
  if (!bias_relu_supported(rows, C)) return 0;
  return (size_t)backward_blocks(rows, C) * (size_t)C * sizeof(float);
}

void bias_relu_backward_bf16(const void* dy, const void* y, void* dz, float* db, int64_t rows, int C, void* scratch,
                             cudaStream_t stream) {
  BAGUA_CHECK(bias_relu_supported(rows, C) && (uintptr_t)dy % 16 == 0 && (uintptr_t)y % 16 == 0 &&
                  (uintptr_t)dz % 16 == 0 && scratch != nullptr,
              Tensor, "fused bias+ReLU backward: unsupported shape [" << rows << ", " << C << "] or unaligned buffers");
  const int blocks = backward_blocks(rows, C);
  bias_relu_backward_kernel<<<blocks, kThreads, 0, stream>>>((const uint4*)dy, (const uint4*)y, (uint4*)dz,
                                                             (float*)scratch, rows, C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  bias_grad_finish_kernel<<<(C + 127) / 128, 128, 0, stream>>>((const float*)scratch, db, blocks, C);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

void maxpool2x2_forward_bf16(const void* x, void* y, int64_t N, int64_t H, int64_t W, int C, cudaStream_t stream) {
  BAGUA_CHECK(maxpool2x2_supported(N, H, W, C) && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0, Tensor,
              "fused max-pool: unsupported shape [" << N << ", " << H << ", " << W << ", " << C << "] or unaligned buffers");
  const int64_t nvec_out = N * (H / 2) * (W / 2) * (C / 8);
  maxpool2x2_forward_kernel<<<pool_grid(nvec_out), kThreads, 0, stream>>>((const uint4*)x, (uint4*)y, nvec_out, W / 2, W,
                                                                          C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

void maxpool2x2_backward_bf16(const void* x, const void* dy, void* dx, int64_t N, int64_t H, int64_t W, int C,
                              cudaStream_t stream) {
  BAGUA_CHECK(maxpool2x2_supported(N, H, W, C) && (uintptr_t)x % 16 == 0 && (uintptr_t)dy % 16 == 0 &&
                  (uintptr_t)dx % 16 == 0,
              Tensor,
              "fused max-pool backward: unsupported shape [" << N << ", " << H << ", " << W << ", " << C
                                                             << "] or unaligned buffers");
  const int64_t nvec_out = N * (H / 2) * (W / 2) * (C / 8);
  maxpool2x2_backward_kernel<<<pool_grid(nvec_out), kThreads, 0, stream>>>((const uint4*)x, (const uint4*)dy, (uint4*)dx,
                                                                           nvec_out, W / 2, W, C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

void bias_relu_pool_bf16(void* y, void* p, const void* bias, int64_t N, int64_t H, int64_t W, int C, cudaStream_t stream) {
  BAGUA_CHECK(bias_relu_supported(N * H * W, C) && maxpool2x2_supported(N, H, W, C) && (uintptr_t)y % 16 == 0 &&
                  (uintptr_t)p % 16 == 0,
              Tensor,
              "fused bias+ReLU+pool: unsupported shape [" << N << ", " << H << ", " << W << ", " << C
                                                          << "] or unaligned buffers");
  const int64_t pooled_pixels = N * (H / 2) * (W / 2);
  bias_relu_pool_kernel<<<pool_grid(pooled_pixels * (C / 8)), kThreads, 0, stream>>>(
      (uint4*)y, (uint4*)p, (const __nv_bfloat16*)bias, pooled_pixels, W / 2, W, C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

void bias_relu_pool_backward_bf16(const void* dp, const void* y, void* dz, float* db, int64_t N, int64_t H, int64_t W,
                                  int C, void* scratch, cudaStream_t stream) {
  BAGUA_CHECK(bias_relu_supported(N * H * W, C) && maxpool2x2_supported(N, H, W, C) && (uintptr_t)dp % 16 == 0 &&
                  (uintptr_t)y % 16 == 0 && (uintptr_t)dz % 16 == 0 && scratch != nullptr,
              Tensor,
              "fused bias+ReLU+pool backward: unsupported shape [" << N << ", " << H << ", " << W << ", " << C
                                                                   << "] or unaligned buffers");
  const int64_t pooled_rows = N * (H / 2) * (W / 2);
  const int blocks = backward_blocks(pooled_rows, C);
  bias_relu_pool_backward_kernel<<<blocks, kThreads, 0, stream>>>((const uint4*)dp, (const uint4*)y, (uint4*)dz,
                                                                  (float*)scratch, pooled_rows, W / 2, W, C / 8);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  bias_grad_finish_kernel<<<(C + 127) / 128, 128, 0, stream>>>((const float*)scratch, db, blocks, C);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace model_ops
}  // namespace bagua
