// Host restatement of every tensor kernel plus the device dispatch.
//
// These loops define the numerics the sm_100a kernels are tested against, and they
// are what the CPU (gloo) backend executes.  MinMaxUInt8 follows the reference's
// anchored grid exactly (bagua-core-internal/kernels/bagua_kernels.cu:10,411-432,
// 465-467): scale = 255/(max-min+1e-7), upper = rint(max*scale), lower = upper-255,
// q = min(rint(x*scale), upper) - lower, x' = (q+lower)/scale.
#include <algorithm>
#include <cmath>
#include <limits>

#include "kernels.h"
#include "kernels_impl.h"

namespace bagua {
namespace kernels {

namespace {

inline float bf16_to_float(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t float_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  uint32_t rounding = 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)((u + rounding) >> 16);
}

template <DType D>
struct Elem;
template <>
struct Elem<DType::F32> {
  using T = float;
  static float ld(const T* p) { return *p; }
  static void st(T* p, float v) { *p = v; }
};
template <>
struct Elem<DType::F16> {
  using T = _Float16;
  static float ld(const T* p) { return (float)*p; }
  static void st(T* p, float v) { *p = (_Float16)v; }
};
template <>
struct Elem<DType::BF16> {
  using T = uint16_t;
  static float ld(const T* p) { return bf16_to_float(*p); }
  static void st(T* p, float v) { *p = float_to_bf16(v); }
};

template <typename F>
void dispatch_float(DType dt, F&& f) {
  switch (dt) {
    case DType::F32: f(Elem<DType::F32>{}); return;
    case DType::F16: f(Elem<DType::F16>{}); return;
    case DType::BF16: f(Elem<DType::BF16>{}); return;
    default:
      throw BaguaError(ErrorKind::Tensor, std::string("kernel does not support dtype ") + dtype_name(dt));
  }
}

template <typename E, typename F>
void map2(void* x, const void* y, int64_t n, F&& f) {
  auto* xp = (typename E::T*)x;
  auto* yp = (const typename E::T*)y;
  for (int64_t i = 0; i < n; ++i) E::st(xp + i, f(E::ld(xp + i), E::ld(yp + i)));
}

}  // namespace

MinMaxGrid minmax_grid(float mn, float mx) {
  const float eps = 1e-7f;
  float denom = (mx - mn) + eps;
  MinMaxGrid g;
  g.scale = (float)(255.0 / (double)denom);
  g.upper = rintf(mx * g.scale);
  g.lower = (float)((double)g.upper - 255.0);
  return g;
}

size_t compressed_buffer_size(int n_chunks, int64_t chunk_size, DType dt) {
  if (dt != DType::F32 && dt != DType::F16 && dt != DType::BF16)
    throw BaguaError(ErrorKind::Tensor, "MinMaxUInt8 compresses floating tensors only");
  return align_up((size_t)chunk_size * (size_t)n_chunks, 32) + (size_t)kCompressHeaderBytes * (size_t)n_chunks;
}

namespace cpu {

void divide_inplace(void* x, DType dt, int64_t n, float d) {
  dispatch_float(dt, [&](auto e) {
    using E = decltype(e);
    auto* p = (typename E::T*)x;
    for (int64_t i = 0; i < n; ++i) E::st(p + i, E::ld(p + i) / d);
  });
}
void add_inplace(void* x, const void* y, DType dt, int64_t n) {
  dispatch_float(dt, [&](auto e) { map2<decltype(e)>(x, y, n, [](float a, float b) { return a + b; }); });
}
void subtract_inplace(void* x, const void* y, DType dt, int64_t n) {
  dispatch_float(dt, [&](auto e) { map2<decltype(e)>(x, y, n, [](float a, float b) { return a - b; }); });
}
void addmul_inplace(void* x, const void* y, float factor, DType dt, int64_t n) {
  dispatch_float(dt, [&](auto e) {
    map2<decltype(e)>(x, y, n, [factor](float a, float b) { return a + b * factor; });
  });
}
void average_inplace(void* x, const void* y, DType dt, int64_t n) {
  dispatch_float(dt, [&](auto e) {
    map2<decltype(e)>(x, y, n, [](float a, float b) { return (a + b) / 2.0f; });
  });
}
void async_model_average(float* t, const float* reduced, const float* copy, float nranks, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    // A compare-and-swap loop keeps the update a single RMW against a concurrently
    // training thread.
    const float delta = reduced[i] / nranks - copy[i];
    uint32_t* word = reinterpret_cast<uint32_t*>(t + i);
    uint32_t old_bits = __atomic_load_n(word, __ATOMIC_RELAXED);
    for (;;) {
      float old_val;
      std::memcpy(&old_val, &old_bits, 4);
      const float new_val = old_val + delta;
      uint32_t new_bits;
      std::memcpy(&new_bits, &new_val, 4);
      if (__atomic_compare_exchange_n(word, &old_bits, new_bits, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) break;
    }
  }
}

void reduce_chunk_inplace(void* x, DType dt, int64_t chunk, int n_chunks, int target, bool average) {
  dispatch_float(dt, [&](auto e) {
    using E = decltype(e);
    auto* p = (typename E::T*)x;
    for (int64_t i = 0; i < chunk; ++i) {
      float s = 0.f;
      for (int c = 0; c < n_chunks; ++c) s += E::ld(p + (int64_t)c * chunk + i);
      if (average) s /= (float)n_chunks;
      E::st(p + (int64_t)target * chunk + i, s);
    }
  });
}

void compress_minmax_u8(const void* in, DType dt, int64_t num_real, int64_t chunk, int n_chunks, uint8_t* out,
                        size_t out_bytes, int target) {
  const size_t off = out_bytes / (size_t)n_chunks;
  dispatch_float(dt, [&](auto e) {
    using E = decltype(e);
    const auto* p = (const typename E::T*)in;
    for (int c = 0; c < n_chunks; ++c) {
      if (target >= 0 && c != target) continue;
      int64_t real = std::min<int64_t>(std::max<int64_t>(num_real - (int64_t)c * chunk, 0), chunk);
      float mn = 0.f, mx = 0.f;
      if (real > 0) {
        mn = std::numeric_limits<float>::infinity();
        mx = -mn;
        for (int64_t i = 0; i < real; ++i) {
          float v = E::ld(p + (int64_t)c * chunk + i);
          mn = std::min(mn, v);
          mx = std::max(mx, v);
        }
      }
      uint8_t* base = out + (size_t)c * off;
      // header is stored in the tensor dtype; quantise with the rounded values so
      // that sender and receiver derive the same grid.
      auto* hdr = (typename E::T*)base;
      E::st(hdr, mn);
      E::st(hdr + 1, mx);
      MinMaxGrid g = minmax_grid(E::ld(hdr), E::ld(hdr + 1));
      uint8_t* q = base + kCompressHeaderBytes;
      for (int64_t i = 0; i < chunk; ++i) {
        float level = rintf(E::ld(p + (int64_t)c * chunk + i) * g.scale);
        level = std::min(level, g.upper);
        float r = level - g.lower;
        // saturating conversion (padding beyond the real range may fall below min)
        r = std::min(std::max(r, 0.f), 255.f);
        q[i] = (uint8_t)r;
      }
    }
  });
}

void decompress_minmax_u8(const uint8_t* in, size_t in_bytes, int64_t chunk, int n_chunks, void* out, DType dt) {
  const size_t off = in_bytes / (size_t)n_chunks;
  dispatch_float(dt, [&](auto e) {
    using E = decltype(e);
    auto* o = (typename E::T*)out;
    for (int c = 0; c < n_chunks; ++c) {
      const uint8_t* base = in + (size_t)c * off;
      const auto* hdr = (const typename E::T*)base;
      MinMaxGrid g = minmax_grid(E::ld(hdr), E::ld(hdr + 1));
      const uint8_t* q = base + kCompressHeaderBytes;
      for (int64_t i = 0; i < chunk; ++i) E::st(o + (int64_t)c * chunk + i, ((float)q[i] + g.lower) / g.scale);
    }
  });
}

void sgd_momentum_flat(float* p, const float* g, float* buf, int64_t n, float lr, float momentum, float dampening,
                       float wd, bool nesterov, bool first_step) {
  for (int64_t i = 0; i < n; ++i) {
    float d = g[i] + wd * p[i];
    if (momentum != 0.f) {
      float b = first_step ? d : momentum * buf[i] + (1.f - dampening) * d;
      buf[i] = b;
      d = nesterov ? d + momentum * b : b;
    }
    p[i] -= lr * d;
  }
}

void sgd_momentum_flat_shadow(float* p, const float* g, float* buf, void* shadow, int64_t n, float lr, float momentum,
                              float dampening, float wd, bool nesterov, bool first_step) {
  sgd_momentum_flat(p, g, buf, n, lr, momentum, dampening, wd, nesterov, first_step);
  uint16_t* h = static_cast<uint16_t*>(shadow);
  for (int64_t i = 0; i < n; ++i) h[i] = float_to_bf16(p[i]);
}

}  // namespace cpu

// ---------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------
void divide_inplace(void* x, DType dt, int64_t n, float d, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::divide_inplace(x, dt, n, d, c.stream) : cpu::divide_inplace(x, dt, n, d);
}
void add_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::add_inplace(x, y, dt, n, c.stream) : cpu::add_inplace(x, y, dt, n);
}
void subtract_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::subtract_inplace(x, y, dt, n, c.stream) : cpu::subtract_inplace(x, y, dt, n);
}
void addmul_inplace(void* x, const void* y, float f, DType dt, int64_t n, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::addmul_inplace(x, y, f, dt, n, c.stream) : cpu::addmul_inplace(x, y, f, dt, n);
}
void average_inplace(void* x, const void* y, DType dt, int64_t n, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::average_inplace(x, y, dt, n, c.stream) : cpu::average_inplace(x, y, dt, n);
}
void async_model_average(float* t, const float* r, const float* cp, float nranks, int64_t n, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::async_model_average(t, r, cp, nranks, n, c.stream)
              : cpu::async_model_average(t, r, cp, nranks, n);
}
void copy_bytes(void* dst, const void* src, size_t bytes, const Ctx& c) {
  if (bytes == 0 || dst == src) return;
  if (c.is_cuda())
    cuda::copy_bytes(dst, src, bytes, c.stream);
  else
    std::memmove(dst, src, bytes);
}
void multi_copy(const MultiCopySeg* segs, int nseg, void* flat, size_t total_bytes, bool gather, const Ctx& c) {
  if (nseg <= 0 || total_bytes == 0) return;
  if (c.is_cuda()) {
    cuda::multi_copy(segs, nseg, flat, total_bytes, gather, c.stream);
    return;
  }
  for (int k = 0; k < nseg; ++k) {
    char* f = (char*)flat + segs[k].offset;
    if (gather)
      std::memmove(f, segs[k].ptr, segs[k].bytes);
    else
      std::memmove(segs[k].ptr, f, segs[k].bytes);
  }
}
void reduce_chunk_inplace(void* x, DType dt, int64_t chunk, int n_chunks, int target, bool average, const Ctx& c) {
  if (chunk <= 0) return;
  BAGUA_CHECK(target >= 0 && target < n_chunks, Tensor, "reduce_chunk_inplace: target chunk out of range");
  c.is_cuda() ? cuda::reduce_chunk_inplace(x, dt, chunk, n_chunks, target, average, c.stream)
              : cpu::reduce_chunk_inplace(x, dt, chunk, n_chunks, target, average);
}
size_t compress_scratch_bytes(int n_chunks, int64_t chunk_size) { return cuda::compress_scratch_bytes(n_chunks, chunk_size); }

void compress_minmax_u8(const void* in, DType dt, int64_t num_real, int64_t chunk, int n_chunks, uint8_t* out,
                        size_t out_bytes, int target, void* scratch, size_t scratch_bytes, const Ctx& c) {
  BAGUA_CHECK(out_bytes >= compressed_buffer_size(n_chunks, chunk, dt), Tensor, "compress: output buffer too small");
  BAGUA_CHECK(target < n_chunks, Tensor, "compress: target chunk out of range");
  if (chunk <= 0) return;
  if (c.is_cuda())
    cuda::compress_minmax_u8(in, dt, num_real, chunk, n_chunks, out, out_bytes, target, scratch, scratch_bytes,
                             c.stream);
  else
    cpu::compress_minmax_u8(in, dt, num_real, chunk, n_chunks, out, out_bytes, target);
}
void decompress_minmax_u8(const uint8_t* in, size_t in_bytes, int64_t chunk, int n_chunks, void* out, DType dt,
                          const Ctx& c) {
  BAGUA_CHECK(in_bytes >= compressed_buffer_size(n_chunks, chunk, dt), Tensor, "decompress: input buffer too small");
  if (chunk <= 0) return;
  c.is_cuda() ? cuda::decompress_minmax_u8(in, in_bytes, chunk, n_chunks, out, dt, c.stream)
              : cpu::decompress_minmax_u8(in, in_bytes, chunk, n_chunks, out, dt);
}
void sgd_momentum_flat(float* p, const float* g, float* buf, int64_t n, float lr, float momentum, float dampening,
                       float wd, bool nesterov, bool first_step, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda() ? cuda::sgd_momentum_flat(p, g, buf, n, lr, momentum, dampening, wd, nesterov, first_step, c.stream)
              : cpu::sgd_momentum_flat(p, g, buf, n, lr, momentum, dampening, wd, nesterov, first_step);
}

void sgd_momentum_flat_shadow(float* p, const float* g, float* buf, void* shadow, int64_t n, float lr, float momentum,
                              float dampening, float wd, bool nesterov, bool first_step, const Ctx& c) {
  if (n <= 0) return;
  c.is_cuda()
      ? cuda::sgd_momentum_flat_shadow(p, g, buf, shadow, n, lr, momentum, dampening, wd, nesterov, first_step, c.stream)
      : cpu::sgd_momentum_flat_shadow(p, g, buf, shadow, n, lr, momentum, dampening, wd, nesterov, first_step);
}

}  // namespace kernels
}  // namespace bagua
