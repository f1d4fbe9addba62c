// sm_100a element-wise and chunk-reduce kernels.
//
// All are HBM-bound streaming kernels: 16-byte accesses, 64-bit indexing, grid sized as
// a multiple of the 148 SMs, fp32 arithmetic with one rounding on store.  They replace
// the reference's scalar 4-byte grid-stride kernels and its shared-memory tree reduce
// (bagua-core-internal/kernels/bagua_kernels.cu:196-266,373-400).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels_impl.h"

namespace bagua {
namespace kernels {
namespace cuda {

namespace {

constexpr int kThreads = 256;
constexpr int kSMs = 148;

template <typename T>
struct VecTraits;
template <>
struct VecTraits<float> {
  static constexpr int N = 4;
};
template <>
struct VecTraits<__half> {
  static constexpr int N = 8;
};
template <>
struct VecTraits<__nv_bfloat16> {
  static constexpr int N = 8;
};

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
struct alignas(16) Pack {
  T v[VecTraits<T>::N];
};

inline int grid_for(int64_t work_items) {
  int64_t blocks = (work_items + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)kSMs * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// x[i] = op(x[i], y[i]) (y may be null for unary ops)
template <typename T, typename Op, bool kVec>
__global__ void __launch_bounds__(kThreads) ew_kernel(T* __restrict__ x, const T* __restrict__ y, int64_t n, Op op) {
  constexpr int V = VecTraits<T>::N;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if constexpr (kVec) {
    const int64_t nv = n / V;
    auto* xv = reinterpret_cast<Pack<T>*>(x);
    auto* yv = reinterpret_cast<const Pack<T>*>(y);
    for (int64_t i = tid; i < nv; i += stride) {
      Pack<T> a = xv[i];
      Pack<T> b;
      if (y) b = yv[i];
#pragma unroll
      for (int k = 0; k < V; ++k) a.v[k] = from_f<T>(op(to_f(a.v[k]), y ? to_f(b.v[k]) : 0.f));
      xv[i] = a;
    }
    for (int64_t i = nv * V + tid; i < n; i += stride) x[i] = from_f<T>(op(to_f(x[i]), y ? to_f(y[i]) : 0.f));
  } else {
    for (int64_t i = tid; i < n; i += stride) x[i] = from_f<T>(op(to_f(x[i]), y ? to_f(y[i]) : 0.f));
  }
}

template <typename T, typename Op>
void launch_ew(void* x, const void* y, int64_t n, Op op, cudaStream_t s) {
  const bool aligned = ((uintptr_t)x % 16 == 0) && (y == nullptr || (uintptr_t)y % 16 == 0);
  if (aligned) {
    int grid = grid_for(n / VecTraits<T>::N + 1);
    ew_kernel<T, Op, true><<<grid, kThreads, 0, s>>>((T*)x, (const T*)y, n, op);
  } else {
    int grid = grid_for(n);
    ew_kernel<T, Op, false><<<grid, kThreads, 0, s>>>((T*)x, (const T*)y, n, op);
  }
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

template <typename Op>
void dispatch_ew(void* x, const void* y, DType dt, int64_t n, Op op, cudaStream_t s) {
  switch (dt) {
    case DType::F32: launch_ew<float>(x, y, n, op, s); return;
    case DType::F16: launch_ew<__half>(x, y, n, op, s); return;
    case DType::BF16: launch_ew<__nv_bfloat16>(x, y, n, op, s); return;
    default: throw BaguaError(ErrorKind::Tensor, std::string("kernel does not support dtype ") + dtype_name(dt));
  }
}

struct OpDiv {
  float d;
  __device__ float operator()(float a, float) const { return a / d; }
};
struct OpAdd {
  __device__ float operator()(float a, float b) const { return a + b; }
};
struct OpSub {
  __device__ float operator()(float a, float b) const { return a - b; }
};
struct OpAddMul {
  float f;
  __device__ float operator()(float a, float b) const { return a + b * f; }
};
struct OpAvg {
  __device__ float operator()(float a, float b) const { return (a + b) * 0.5f; }
};

__global__ void __launch_bounds__(kThreads)
    async_avg_kernel(float* __restrict__ t, const float* __restrict__ r, const float* __restrict__ cp, float nranks,
                     int64_t n, bool vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t nv = n / 4;
    for (int64_t i = tid; i < nv; i += stride) {
      float4 a = reinterpret_cast<const float4*>(r)[i];
      float4 b = reinterpret_cast<const float4*>(cp)[i];
      float4 d = make_float4(a.x / nranks - b.x, a.y / nranks - b.y, a.z / nranks - b.z, a.w / nranks - b.w);
      // one 16-byte vector reduction instead of four scalar atomics
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(t + 4 * i), "f"(d.x), "f"(d.y), "f"(d.z),
                   "f"(d.w)
                   : "memory");
    }
    for (int64_t i = nv * 4 + tid; i < n; i += stride) atomicAdd(t + i, r[i] / nranks - cp[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride) atomicAdd(t + i, r[i] / nranks - cp[i]);
  }
}

// x as [n_chunks][chunk]; each thread owns V adjacent columns and walks the chunks.
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads)
    reduce_chunk_kernel(T* __restrict__ x, int64_t chunk, int n_chunks, int target, float mul) {
  constexpr int V = VecTraits<T>::N;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if constexpr (kVec) {
    const int64_t nv = chunk / V;
    for (int64_t i = tid; i < nv; i += stride) {
      float acc[V];
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] = 0.f;
      for (int c = 0; c < n_chunks; ++c) {
        Pack<T> a = reinterpret_cast<const Pack<T>*>(x + (int64_t)c * chunk)[i];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] += to_f(a.v[k]);
      }
      Pack<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(acc[k] * mul);
      reinterpret_cast<Pack<T>*>(x + (int64_t)target * chunk)[i] = o;
    }
  } else {
    for (int64_t i = tid; i < chunk; i += stride) {
      float acc = 0.f;
      for (int c = 0; c < n_chunks; ++c) acc += to_f(x[(int64_t)c * chunk + i]);
      x[(int64_t)target * chunk + i] = from_f<T>(acc * mul);
    }
  }
}

template <typename T>
void launch_reduce_chunk(void* x, int64_t chunk, int n_chunks, int target, bool average, cudaStream_t s) {
  constexpr int V = VecTraits<T>::N;
  // exact division keeps the mean bit-identical to sum / n for power-of-two n and within
  // 1 ulp otherwise; the host oracle divides, tests compare with a tolerance.
  const float mul = average ? 1.0f / (float)n_chunks : 1.0f;
  const bool vec = ((uintptr_t)x % 16 == 0) && (chunk % V == 0);
  if (vec) {
    reduce_chunk_kernel<T, true><<<grid_for(chunk / V), kThreads, 0, s>>>((T*)x, chunk, n_chunks, target, mul);
  } else {
    reduce_chunk_kernel<T, false><<<grid_for(chunk), kThreads, 0, s>>>((T*)x, chunk, n_chunks, target, mul);
  }
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

__global__ void __launch_bounds__(kThreads)
    sgd_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ buf, int64_t n, float lr,
               float momentum, float dampening, float wd, bool nesterov, bool first, bool vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  auto upd = [&](float& pv, float gv, float& bv) {
    float d = gv + wd * pv;
    if (momentum != 0.f) {
      float b = first ? d : momentum * bv + (1.f - dampening) * d;
      bv = b;
      d = nesterov ? d + momentum * b : b;
    }
    pv -= lr * d;
  };
  if (vec) {
    const int64_t nv = n / 4;
    for (int64_t i = tid; i < nv; i += stride) {
      float4 pv = reinterpret_cast<float4*>(p)[i];
      float4 gv = reinterpret_cast<const float4*>(g)[i];
      float4 bv = (momentum != 0.f && !first) ? reinterpret_cast<float4*>(buf)[i] : make_float4(0, 0, 0, 0);
      upd(pv.x, gv.x, bv.x);
      upd(pv.y, gv.y, bv.y);
      upd(pv.z, gv.z, bv.z);
      upd(pv.w, gv.w, bv.w);
      reinterpret_cast<float4*>(p)[i] = pv;
      if (momentum != 0.f) reinterpret_cast<float4*>(buf)[i] = bv;
    }
    for (int64_t i = nv * 4 + tid; i < n; i += stride) {
      float bv = (momentum != 0.f && !first) ? buf[i] : 0.f;
      upd(p[i], g[i], bv);
      if (momentum != 0.f) buf[i] = bv;
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      float bv = (momentum != 0.f && !first) ? buf[i] : 0.f;
      upd(p[i], g[i], bv);
      if (momentum != 0.f) buf[i] = bv;
    }
  }
}

// The same step with a bf16 copy of every updated parameter (a kernel of its own, so that the
// plain step keeps its code): 4 parameters per thread-iteration, their bf16 values go out as
// one 8-byte store.
__global__ void __launch_bounds__(kThreads)
    sgd_shadow_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ buf,
                      __nv_bfloat16* __restrict__ shadow, int64_t n, float lr, float momentum, float dampening, float wd,
                      bool nesterov, bool first, bool vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  auto upd = [&](float& pv, float gv, float& bv) {
    float d = gv + wd * pv;
    if (momentum != 0.f) {
      float b = first ? d : momentum * bv + (1.f - dampening) * d;
      bv = b;
      d = nesterov ? d + momentum * b : b;
    }
    pv -= lr * d;
  };
  auto one = [&](int64_t i) {
    float bv = (momentum != 0.f && !first) ? buf[i] : 0.f;
    upd(p[i], g[i], bv);
    if (momentum != 0.f) buf[i] = bv;
    shadow[i] = __float2bfloat16_rn(p[i]);
  };
  if (vec) {
    const int64_t nv = n / 4;
    for (int64_t i = tid; i < nv; i += stride) {
      float4 pv = reinterpret_cast<float4*>(p)[i];
      float4 gv = reinterpret_cast<const float4*>(g)[i];
      float4 bv = (momentum != 0.f && !first) ? reinterpret_cast<float4*>(buf)[i] : make_float4(0, 0, 0, 0);
      upd(pv.x, gv.x, bv.x);
      upd(pv.y, gv.y, bv.y);
      upd(pv.z, gv.z, bv.z);
      upd(pv.w, gv.w, bv.w);
      reinterpret_cast<float4*>(p)[i] = pv;
      if (momentum != 0.f) reinterpret_cast<float4*>(buf)[i] = bv;
      uint2 h;
      *reinterpret_cast<__nv_bfloat162*>(&h.x) = __floats2bfloat162_rn(pv.x, pv.y);
      *reinterpret_cast<__nv_bfloat162*>(&h.y) = __floats2bfloat162_rn(pv.z, pv.w);
      reinterpret_cast<uint2*>(shadow)[i] = h;
    }
    for (int64_t i = nv * 4 + tid; i < n; i += stride) one(i);
  } else {
    for (int64_t i = tid; i < n; i += stride) one(i);
  }
}

}  // namespace

void divide_inplace(void* x, DType dt, int64_t n, float d, cudaStream_t s) {
  dispatch_ew(x, nullptr, dt, n, OpDiv{d}, s);
}
void add_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s) { dispatch_ew(x, y, dt, n, OpAdd{}, s); }
void subtract_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s) {
  dispatch_ew(x, y, dt, n, OpSub{}, s);
}
void addmul_inplace(void* x, const void* y, float f, DType dt, int64_t n, cudaStream_t s) {
  dispatch_ew(x, y, dt, n, OpAddMul{f}, s);
}
void average_inplace(void* x, const void* y, DType dt, int64_t n, cudaStream_t s) {
  dispatch_ew(x, y, dt, n, OpAvg{}, s);
}
void async_model_average(float* t, const float* r, const float* cp, float nranks, int64_t n, cudaStream_t s) {
  const bool vec = ((uintptr_t)t % 16 == 0) && ((uintptr_t)r % 16 == 0) && ((uintptr_t)cp % 16 == 0);
  async_avg_kernel<<<grid_for(vec ? n / 4 + 1 : n), kThreads, 0, s>>>(t, r, cp, nranks, n, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}
void copy_bytes(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  BAGUA_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s));
}
void reduce_chunk_inplace(void* x, DType dt, int64_t chunk, int n_chunks, int target, bool average, cudaStream_t s) {
  switch (dt) {
    case DType::F32: launch_reduce_chunk<float>(x, chunk, n_chunks, target, average, s); return;
    case DType::F16: launch_reduce_chunk<__half>(x, chunk, n_chunks, target, average, s); return;
    case DType::BF16: launch_reduce_chunk<__nv_bfloat16>(x, chunk, n_chunks, target, average, s); return;
    default: throw BaguaError(ErrorKind::Tensor, std::string("reduce_chunk: unsupported dtype ") + dtype_name(dt));
  }
}
void sgd_momentum_flat(float* p, const float* g, float* buf, int64_t n, float lr, float momentum, float dampening,
                       float wd, bool nesterov, bool first_step, cudaStream_t s) {
  const bool vec = ((uintptr_t)p % 16 == 0) && ((uintptr_t)g % 16 == 0) && ((uintptr_t)buf % 16 == 0);
  sgd_kernel<<<grid_for(vec ? n / 4 + 1 : n), kThreads, 0, s>>>(p, g, buf, n, lr, momentum, dampening, wd, nesterov,
                                                                 first_step, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

void sgd_momentum_flat_shadow(float* p, const float* g, float* buf, void* shadow, int64_t n, float lr, float momentum,
                              float dampening, float wd, bool nesterov, bool first_step, cudaStream_t s) {
  const bool vec = ((uintptr_t)p % 16 == 0) && ((uintptr_t)g % 16 == 0) && ((uintptr_t)buf % 16 == 0) &&
                   ((uintptr_t)shadow % 8 == 0);
  sgd_shadow_kernel<<<grid_for(vec ? n / 4 + 1 : n), kThreads, 0, s>>>(p, g, buf, (__nv_bfloat16*)shadow, n, lr, momentum,
                                                                        dampening, wd, nesterov, first_step, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace cuda
}  // namespace kernels
}  // namespace bagua
