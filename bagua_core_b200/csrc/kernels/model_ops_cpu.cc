// Host restatement of the fused model kernels (model_ops.cu): the same math as plain loops over
// bf16 data, used for CPU tensors.  It is the oracle for the CUDA kernels and lets the autograd
// glue around them (bagua_core_b200/ops/fused_conv.py) be tested without a GPU.
#include <cmath>
#include <cstring>
#include <vector>

#include "model_ops.h"

namespace bagua {
namespace model_ops {

namespace {

inline float bf16_to_float(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
// round to nearest even, like __float2bfloat16_rn
inline uint16_t float_to_bf16(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);  // NaN stays NaN
  const uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return (uint16_t)(bits >> 16);
}

}  // namespace

bool bias_relu_supported(int64_t rows, int C) {
  if (rows <= 0 || C < 8 || C > 2048 || C % 8 != 0) return false;
  const int cgroups = C / 8;
  return kBlockThreads % cgroups == 0;  // the backward's thread layout: [rows per iteration][C / 8]
}

bool maxpool2x2_supported(int64_t N, int64_t H, int64_t W, int C) {
  return N > 0 && H >= 2 && W >= 2 && H % 2 == 0 && W % 2 == 0 && C >= 8 && C % 8 == 0;
}

void bias_relu_inplace_bf16_host(void* z, const void* bias, int64_t rows, int C) {
  uint16_t* p = static_cast<uint16_t*>(z);
  const uint16_t* b = static_cast<const uint16_t*>(bias);
  for (int64_t r = 0; r < rows; ++r)
    for (int c = 0; c < C; ++c) {
      const float v = bf16_to_float(p[r * C + c]) + bf16_to_float(b[c]);
      p[r * C + c] = float_to_bf16(v > 0.f ? v : 0.f);
    }
}

void bias_relu_backward_bf16_host(const void* dy, const void* y, void* dz, float* db, int64_t rows, int C) {
  const uint16_t* g = static_cast<const uint16_t*>(dy);
  const uint16_t* o = static_cast<const uint16_t*>(y);
  uint16_t* out = static_cast<uint16_t*>(dz);
  std::vector<double> acc((size_t)C, 0.0);
  for (int64_t r = 0; r < rows; ++r)
    for (int c = 0; c < C; ++c) {
      const float v = bf16_to_float(o[r * C + c]) > 0.f ? bf16_to_float(g[r * C + c]) : 0.f;
      out[r * C + c] = float_to_bf16(v);
      acc[(size_t)c] += (double)v;
    }
  for (int c = 0; c < C; ++c) db[c] = (float)acc[(size_t)c];
}

void maxpool2x2_forward_bf16_host(const void* x, void* y, int64_t N, int64_t H, int64_t W, int C) {
  const uint16_t* in = static_cast<const uint16_t*>(x);
  uint16_t* out = static_cast<uint16_t*>(y);
  const int64_t Ho = H / 2, Wo = W / 2;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t ho = 0; ho < Ho; ++ho)
      for (int64_t wo = 0; wo < Wo; ++wo)
        for (int c = 0; c < C; ++c) {
          const int64_t base = ((n * H + 2 * ho) * W + 2 * wo) * C + c;
          const float a = bf16_to_float(in[base]), b = bf16_to_float(in[base + C]);
          const float cc = bf16_to_float(in[base + W * C]), d = bf16_to_float(in[base + W * C + C]);
          out[((n * Ho + ho) * Wo + wo) * C + c] = float_to_bf16(std::fmax(std::fmax(a, b), std::fmax(cc, d)));
        }
}

void maxpool2x2_backward_bf16_host(const void* x, const void* dy, void* dx, int64_t N, int64_t H, int64_t W, int C) {
  const uint16_t* in = static_cast<const uint16_t*>(x);
  const uint16_t* g = static_cast<const uint16_t*>(dy);
  uint16_t* out = static_cast<uint16_t*>(dx);
  const int64_t Ho = H / 2, Wo = W / 2;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t ho = 0; ho < Ho; ++ho)
      for (int64_t wo = 0; wo < Wo; ++wo)
        for (int c = 0; c < C; ++c) {
          const int64_t base = ((n * H + 2 * ho) * W + 2 * wo) * C + c;
          const int64_t off[4] = {0, C, W * C, W * C + C};
          int idx = 0;
          float m = bf16_to_float(in[base]);
          for (int k = 1; k < 4; ++k) {
            const float v = bf16_to_float(in[base + off[k]]);
            if (v > m) {  // a later element wins only if strictly larger
              m = v;
              idx = k;
            }
          }
          const uint16_t grad = g[((n * Ho + ho) * Wo + wo) * C + c];
          for (int k = 0; k < 4; ++k) out[base + off[k]] = k == idx ? grad : (uint16_t)0;
        }
}

// The pooled pair is, by definition, the composition of the two single steps.
void bias_relu_pool_bf16_host(void* y, void* p, const void* bias, int64_t N, int64_t H, int64_t W, int C) {
  bias_relu_inplace_bf16_host(y, bias, N * H * W, C);
  maxpool2x2_forward_bf16_host(y, p, N, H, W, C);
}

void bias_relu_pool_backward_bf16_host(const void* dp, const void* y, void* dz, float* db, int64_t N, int64_t H,
                                       int64_t W, int C) {
  std::vector<uint16_t> dy((size_t)(N * H * W * C));
  maxpool2x2_backward_bf16_host(y, dp, dy.data(), N, H, W, C);
  bias_relu_backward_bf16_host(dy.data(), y, dz, db, N * H * W, C);
}

}  // namespace model_ops
}  // namespace bagua
