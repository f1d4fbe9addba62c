// Fused element-wise kernels for the benchmark models' convolution blocks (sm_100a).
//
// A VGG-style block is convolution → bias → ReLU.  The framework runs the bias/ReLU part as
// separate passes over the activation (forward: add, clamp; backward: ReLU mask, then a
// column reduction for the bias gradient, which alone took 12 % of a VGG-16 step on a B200).
// These kernels do each direction in one pass over a channels-last activation viewed as a
// row-major [rows = N·H·W, C] matrix of bf16:
//   forward   y = max(z + bias, 0), in place on the convolution's output;
//   backward  dz = dy · [y > 0] and db[c] = Σ_rows dz[row, c] (fp32 accumulation, fixed
//             summation order, no atomics), from one read of dy and y.
// The pooling layers between the blocks get the same treatment (see below).
// No counterpart in the reference, which has no model code.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace bagua {
namespace model_ops {

// Threads per block of the CUDA kernels.
constexpr int kBlockThreads = 256;

// C must be a multiple of 8, 8 <= C <= 2048, C / 8 a divisor of kBlockThreads; pointers 16-byte aligned.
bool bias_relu_supported(int64_t rows, int C);

// z: [rows, C] bf16 (in place), bias: [C] bf16.
void bias_relu_inplace_bf16(void* z, const void* bias, int64_t rows, int C, cudaStream_t stream);

// Bytes of scratch (per-block partial sums) the backward needs for this shape.
size_t bias_relu_backward_scratch_bytes(int64_t rows, int C);

// dy, y, dz: [rows, C] bf16 (dz may alias dy); db: [C] fp32; scratch as sized above.
void bias_relu_backward_bf16(const void* dy, const void* y, void* dz, float* db, int64_t rows, int C, void* scratch,
                             cudaStream_t stream);

// ---- 2x2 / stride-2 max pooling on channels-last bf16 activations ---------------------
// x: [N, H, W, C] (H, W even, C a multiple of 8), y: [N, H/2, W/2, C].  The forward stores no
// index tensor; the backward recomputes each window's arg-max from x (first maximum in
// (h, w) scan order, like the framework's kernel) and writes every element of dx exactly
// once, so dx needs no zero-fill and no atomics.
bool maxpool2x2_supported(int64_t N, int64_t H, int64_t W, int C);
void maxpool2x2_forward_bf16(const void* x, void* y, int64_t N, int64_t H, int64_t W, int C, cudaStream_t stream);
void maxpool2x2_backward_bf16(const void* x, const void* dy, void* dx, int64_t N, int64_t H, int64_t W, int C,
                              cudaStream_t stream);

// ---- bias + ReLU followed by 2x2 pooling, as one forward and one backward pass ------------
// y: [N, H, W, C] convolution output, overwritten with max(y + bias, 0); p: [N, H/2, W/2, C].
// Needs both bias_relu_supported(N*H*W, C) and maxpool2x2_supported(N, H, W, C).
void bias_relu_pool_bf16(void* y, void* p, const void* bias, int64_t N, int64_t H, int64_t W, int C, cudaStream_t stream);
// dp: [N, H/2, W/2, C]; y as written by the forward; dz: [N, H, W, C] (every element written);
// db: [C] fp32; scratch of bias_relu_backward_scratch_bytes(N*(H/2)*(W/2), C) bytes.
void bias_relu_pool_backward_bf16(const void* dp, const void* y, void* dz, float* db, int64_t N, int64_t H, int64_t W,
                                  int C, void* scratch, cudaStream_t stream);

// ---- host restatements (model_ops_cpu.cc): same arguments, host pointers, any C ----------
void bias_relu_inplace_bf16_host(void* z, const void* bias, int64_t rows, int C);
void bias_relu_backward_bf16_host(const void* dy, const void* y, void* dz, float* db, int64_t rows, int C);
void maxpool2x2_forward_bf16_host(const void* x, void* y, int64_t N, int64_t H, int64_t W, int C);
void maxpool2x2_backward_bf16_host(const void* x, const void* dy, void* dx, int64_t N, int64_t H, int64_t W, int C);
void bias_relu_pool_bf16_host(void* y, void* p, const void* bias, int64_t N, int64_t H, int64_t W, int C);
void bias_relu_pool_backward_bf16_host(const void* dp, const void* y, void* dz, float* db, int64_t N, int64_t H,
                                       int64_t W, int C);

}  // namespace model_ops
}  // namespace bagua
