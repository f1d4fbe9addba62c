// Device bodies of the fused model kernels (see model_ops.cu / model_ops.h).  Kept in a header so
// that the same source is compiled by nvcc into the sm_100a kernels and by the host compiler
// (-DBAGUA_HOST_EMULATION, host_emulation.h) into tests/cpp/model_ops_emulation.cc, which runs
// them thread for thread against the host restatement.  Shared memory is handed in by the caller.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "host_emulation.h"

namespace bagua {
namespace model_ops {
namespace bodies {

constexpr int kThreads = 256;
constexpr int kMaxBlocks = 148 * 4;

__device__ __forceinline__ void unpack8(const uint4& x, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 v = __bfloat1622float2(h[k]);
    f[2 * k] = v.x;
    f[2 * k + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return r;
}

// ---- forward ----------------------------------------------------------------------
__device__ __forceinline__ uint4 bias_relu_vec(const uint4& x, const float* b) {
  float f[8];
  unpack8(x, f);
#pragma unroll
  for (int k = 0; k < 8; ++k) f[k] = fmaxf(f[k] + b[k], 0.f);
  return pack8(f);
}

// The 8 bias values of channel group cg.
__device__ __forceinline__ void load_bias8(const __nv_bfloat16* __restrict__ bias, int cg, float (&b)[8]) {
#pragma unroll
  for (int k = 0; k < 8; ++k) b[k] = __bfloat162float(bias[cg * 8 + k]);
}

// cgroups = C / 8 vectors per row.  cgroups divides kThreads, hence the grid stride too, so all
// vectors a thread visits belong to one channel group: its bias stays in registers and the loop
// has no division.
__device__ __forceinline__ void bias_relu_body(uint4* __restrict__ z, const __nv_bfloat16* __restrict__ bias,
                                               int64_t nvec, int cgroups) {
  float bs[8];
  load_bias8(bias, (int)(threadIdx.x % cgroups), bs);
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  for (; v + 3 * stride < nvec; v += 4 * stride) {
    const uint4 a = z[v], b = z[v + stride], c = z[v + 2 * stride], d = z[v + 3 * stride];
    z[v] = bias_relu_vec(a, bs);
    z[v + stride] = bias_relu_vec(b, bs);
    z[v + 2 * stride] = bias_relu_vec(c, bs);
    z[v + 3 * stride] = bias_relu_vec(d, bs);
  }
  for (; v < nvec; v += stride) z[v] = bias_relu_vec(z[v], bs);
}

// ---- backward ---------------------------------------------------------------------
__device__ __forceinline__ uint4 relu_mask_acc(const uint4& dy, const uint4& y, float (&acc)[8]) {
  float g[8], o[8];
  unpack8(dy, g);
  unpack8(y, o);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    g[k] = o[k] > 0.f ? g[k] : 0.f;
    acc[k] += g[k];
  }
  return pack8(g);
}

// Threads are laid out [rows_per_iter][cgroups]: thread (ro, cg) visits rows ro, ro + R, ...
// (R = gridDim.x * rows_per_iter apart) and always the same 8 channels.  cgroups divides kThreads.
__device__ __forceinline__ void bias_relu_backward_body(const uint4* dy, const uint4* __restrict__ y, uint4* dz,
                                                        float* __restrict__ partial, int64_t rows, int cgroups,
                                                        float* s_acc) {
  const int rows_per_iter = kThreads / cgroups;
  const int cg = threadIdx.x % cgroups, ro = threadIdx.x / cgroups;
  const int64_t step = (int64_t)gridDim.x * rows_per_iter;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  int64_t row = (int64_t)blockIdx.x * rows_per_iter + ro;
  for (; row + step < rows; row += 2 * step) {
    const int64_t v0 = row * cgroups + cg, v1 = (row + step) * cgroups + cg;
    const uint4 a0 = dy[v0], b0 = y[v0], a1 = dy[v1], b1 = y[v1];
    dz[v0] = relu_mask_acc(a0, b0, acc);
    dz[v1] = relu_mask_acc(a1, b1, acc);
  }
  for (; row < rows; row += step) {
    const int64_t v0 = row * cgroups + cg;
    dz[v0] = relu_mask_acc(dy[v0], y[v0], acc);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) s_acc[threadIdx.x * 8 + k] = acc[k];
  __syncthreads();
  const int C = cgroups * 8;
  for (int c = threadIdx.x; c < C; c += kThreads) {
    const int g = c >> 3, k = c & 7;
    float s = 0.f;
    for (int r = 0; r < rows_per_iter; ++r) s += s_acc[(r * cgroups + g) * 8 + k];
    partial[(size_t)blockIdx.x * C + c] = s;
  }
}

__device__ __forceinline__ void bias_grad_finish_body(const float* __restrict__ partial, float* __restrict__ db,
                                                      int blocks, int C) {
  const int c = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= C) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[(size_t)b * C + c];
  db[c] = s;
}

// ---- 2x2 / stride-2 max pooling -------------------------------------------------------
// Vector indices are [n][h][w][cg] with cg fastest, so a warp reads whole pixels of contiguous
// channels.  Index arithmetic divides in 32 bits whenever the value fits: the 64-bit division
// costs several times as many instructions, enough to show next to the handful of 16-byte
// accesses a thread makes per output vector.
__device__ __forceinline__ void div_mod(int64_t a, int64_t d, int64_t& quot, int64_t& rem) {
  if (a <= 0xffffffffLL && d <= 0xffffffffLL) {
    const uint32_t a32 = (uint32_t)a, d32 = (uint32_t)d, q32 = a32 / d32;
    quot = q32;
    rem = a32 - q32 * d32;
  } else {
    quot = a / d;
    rem = a - quot * d;
  }
}

struct PoolIndex {
  int64_t x00;  // vector index of the window's top-left input pixel
  int64_t dw, dh;  // vector strides to the right / lower neighbour
};
// Pooled pixel p = (n * Ho + ho) * Wo + wo of an [N, 2 Ho, W, C] input: its window starts at
// input row 2 (n * Ho + ho), column 2 wo, so one division by Wo is all it takes.
__device__ __forceinline__ PoolIndex pool_index(int64_t p, int64_t cg, int64_t Wo, int64_t W, int cgroups) {
  int64_t q, wo;
  div_mod(p, Wo, q, wo);
  PoolIndex r;
  r.dw = cgroups;
  r.dh = W * cgroups;
  r.x00 = (2 * q * W + 2 * wo) * cgroups + cg;
  return r;
}

// One thread per output vector (8 channels of one output pixel); any number of channel groups.
__device__ __forceinline__ void maxpool2x2_forward_body(const uint4* __restrict__ x, uint4* __restrict__ y,
                                                        int64_t nvec_out, int64_t Wo, int64_t W, int cgroups) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec_out; v += stride) {
    int64_t pixel, cg;
    div_mod(v, cgroups, pixel, cg);
    const PoolIndex p = pool_index(pixel, cg, Wo, W, cgroups);
    const uint4 a = x[p.x00], b = x[p.x00 + p.dw], c = x[p.x00 + p.dh], d = x[p.x00 + p.dh + p.dw];
    float fa[8], fb[8], fc[8], fd[8];
    unpack8(a, fa);
    unpack8(b, fb);
    unpack8(c, fc);
    unpack8(d, fd);
#pragma unroll
    for (int k = 0; k < 8; ++k) fa[k] = fmaxf(fmaxf(fa[k], fb[k]), fmaxf(fc[k], fd[k]));
    y[v] = pack8(fa);
  }
}

__device__ __forceinline__ void maxpool2x2_backward_body(const uint4* __restrict__ x, const uint4* __restrict__ dy,
                                                         uint4* __restrict__ dx, int64_t nvec_out, int64_t Wo,
                                                         int64_t W, int cgroups) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec_out; v += stride) {
    int64_t pixel, cg;
    div_mod(v, cgroups, pixel, cg);
    const PoolIndex p = pool_index(pixel, cg, Wo, W, cgroups);
    const uint4 a = x[p.x00], b = x[p.x00 + p.dw], c = x[p.x00 + p.dh], d = x[p.x00 + p.dh + p.dw];
    const uint4 g4 = dy[v];
    float fa[8], fb[8], fc[8], fd[8], g[8];
    unpack8(a, fa);
    unpack8(b, fb);
    unpack8(c, fc);
    unpack8(d, fd);
    unpack8(g4, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // first maximum in scan order (0,0) (0,1) (1,0) (1,1): a later element wins only if strictly larger
      float m = fa[k];
      int idx = 0;
      if (fb[k] > m) {
        m = fb[k];
        idx = 1;
      }
      if (fc[k] > m) {
        m = fc[k];
        idx = 2;
      }
      if (fd[k] > m) idx = 3;
      fa[k] = idx == 0 ? g[k] : 0.f;
      fb[k] = idx == 1 ? g[k] : 0.f;
      fc[k] = idx == 2 ? g[k] : 0.f;
      fd[k] = idx == 3 ? g[k] : 0.f;
    }
    dx[p.x00] = pack8(fa);
    dx[p.x00 + p.dw] = pack8(fb);
    dx[p.x00 + p.dh] = pack8(fc);
    dx[p.x00 + p.dh + p.dw] = pack8(fd);
  }
}

// ---- bias + ReLU with the 2x2 pooling that follows it -----------------------------------
// Forward: y = max(z + bias, 0) in place on the [N, H, W, C] convolution output, and
// p = 2x2 max of y, both from one read of z.  One thread per pooled vector; cgroups divides
// kThreads, so a thread keeps its channel group (and its bias, in registers) and walks pooled
// pixels that are a fixed number apart.
__device__ __forceinline__ void bias_relu_pool_body(uint4* __restrict__ y, uint4* __restrict__ p,
                                                    const __nv_bfloat16* __restrict__ bias, int64_t pooled_pixels,
                                                    int64_t Wo, int64_t W, int cgroups) {
  const int cg = (int)(threadIdx.x % cgroups);
  float b[8];
  load_bias8(bias, cg, b);
  const int64_t pixel_step = (int64_t)gridDim.x * (kThreads / cgroups);
  for (int64_t px = (int64_t)blockIdx.x * (kThreads / cgroups) + threadIdx.x / cgroups; px < pooled_pixels;
       px += pixel_step) {
    const PoolIndex q = pool_index(px, cg, Wo, W, cgroups);
    const uint4 a0 = y[q.x00], a1 = y[q.x00 + q.dw], a2 = y[q.x00 + q.dh], a3 = y[q.x00 + q.dh + q.dw];
    const uint4 r0 = bias_relu_vec(a0, b), r1 = bias_relu_vec(a1, b), r2 = bias_relu_vec(a2, b), r3 = bias_relu_vec(a3, b);
    y[q.x00] = r0;
    y[q.x00 + q.dw] = r1;
    y[q.x00 + q.dh] = r2;
    y[q.x00 + q.dh + q.dw] = r3;
    float f0[8], f1[8], f2[8], f3[8];
    unpack8(r0, f0);
    unpack8(r1, f1);
    unpack8(r2, f2);
    unpack8(r3, f3);
#pragma unroll
    for (int k = 0; k < 8; ++k) f0[k] = fmaxf(fmaxf(f0[k], f1[k]), fmaxf(f2[k], f3[k]));
    p[px * cgroups + cg] = pack8(f0);
  }
}

// Backward of the pair: dz = dp routed to each window's first maximum of y, masked by y > 0,
// zero elsewhere; db[c] = column sums of dz.  Thread (ro, cg) visits pooled pixels ro, ro + R, ...
// and always the same 8 channels, like the un-pooled backward.
__device__ __forceinline__ void bias_relu_pool_backward_body(const uint4* __restrict__ dp, const uint4* __restrict__ y,
                                                             uint4* __restrict__ dz, float* __restrict__ partial,
                                                             int64_t pooled_rows, int64_t Wo, int64_t W, int cgroups,
                                                             float* s_acc) {
  const int rows_per_iter = kThreads / cgroups;
  const int cg = threadIdx.x % cgroups, ro = threadIdx.x / cgroups;
  const int64_t step = (int64_t)gridDim.x * rows_per_iter;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int64_t pr = (int64_t)blockIdx.x * rows_per_iter + ro; pr < pooled_rows; pr += step) {
    const int64_t v = pr * cgroups + cg;
    const PoolIndex q = pool_index(pr, cg, Wo, W, cgroups);
    const uint4 a0 = y[q.x00], a1 = y[q.x00 + q.dw], a2 = y[q.x00 + q.dh], a3 = y[q.x00 + q.dh + q.dw];
    const uint4 g4 = dp[v];
    float f0[8], f1[8], f2[8], f3[8], g[8];
    unpack8(a0, f0);
    unpack8(a1, f1);
    unpack8(a2, f2);
    unpack8(a3, f3);
    unpack8(g4, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float m = f0[k];
      int idx = 0;
      if (f1[k] > m) {
        m = f1[k];
        idx = 1;
      }
      if (f2[k] > m) {
        m = f2[k];
        idx = 2;
      }
      if (f3[k] > m) {
        m = f3[k];
        idx = 3;
      }
      const float gv = m > 0.f ? g[k] : 0.f;  // the ReLU mask of the element the gradient goes to
      acc[k] += gv;
      f0[k] = idx == 0 ? gv : 0.f;
      f1[k] = idx == 1 ? gv : 0.f;
      f2[k] = idx == 2 ? gv : 0.f;
      f3[k] = idx == 3 ? gv : 0.f;
    }
    dz[q.x00] = pack8(f0);
    dz[q.x00 + q.dw] = pack8(f1);
    dz[q.x00 + q.dh] = pack8(f2);
    dz[q.x00 + q.dh + q.dw] = pack8(f3);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) s_acc[threadIdx.x * 8 + k] = acc[k];
  __syncthreads();
  const int C = cgroups * 8;
  for (int c = threadIdx.x; c < C; c += kThreads) {
    const int g = c >> 3, k = c & 7;
    float s = 0.f;
    for (int r = 0; r < rows_per_iter; ++r) s += s_acc[(r * cgroups + g) * 8 + k];
    partial[(size_t)blockIdx.x * C + c] = s;
  }
}

}  // namespace bodies
}  // namespace model_ops
}  // namespace bagua
