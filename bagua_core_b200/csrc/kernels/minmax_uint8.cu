// MinMaxUInt8 compression for sm_100a: per-chunk min/max, quantise, dequantise.
//
// Two launches per compress call regardless of the number of chunks: (1) every block
// reduces a slice of one chunk to a partial {min,max} in scratch; (2) every block first
// folds the partials of its chunk (they sit in L2), derives the grid, and quantises its
// slice with 16-byte loads and stores.  No atomics, no initialisation of scratch, and
// deterministic.  The reference issues two CUB DeviceReduce calls per chunk from a host
// loop (bagua-core-internal/kernels/bagua_kernels.cu:312-371,533-560) and quantises one
// byte per thread (455-479).
//
// Numerics are the reference's anchored grid (see MinMaxGrid in kernels.h); the header
// is stored in the tensor dtype and the grid is derived from the stored (rounded) values
// on both sides.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "kernels_impl.h"
#include "minmax_device.cuh"

namespace bagua {
namespace kernels {
namespace cuda {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxBlocksPerChunk = 1024;

inline int blocks_per_chunk(int n_chunks, int64_t chunk) {
  // ~16 KiB of elements per block, at most ~8 blocks per SM over the whole launch
  int64_t want = (chunk + 4095) / 4096;
  int64_t cap = std::max<int64_t>(1, (148 * 8) / std::max(1, n_chunks));
  int64_t b = std::min<int64_t>(std::min<int64_t>(want, cap), kMaxBlocksPerChunk);
  return (int)std::max<int64_t>(b, 1);
}

// Slice [lo, hi) of a chunk owned by block bx of nb, rounded to 16-element groups.
__device__ __forceinline__ void block_slice(int64_t chunk, int bx, int nb, int64_t& lo, int64_t& hi) {
  int64_t groups = (chunk + 15) / 16;
  int64_t per = (groups + nb - 1) / nb;
  lo = min((int64_t)bx * per * 16, chunk);
  hi = min(lo + per * 16, chunk);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    minmax_partial_kernel(const T* __restrict__ in, int64_t num_real, int64_t chunk, int first_chunk,
                          float2* __restrict__ partial, bool vec) {
  const int c = first_chunk + blockIdx.y;
  int64_t real = num_real - (int64_t)c * chunk;
  real = real < 0 ? 0 : (real > chunk ? chunk : real);
  int64_t lo, hi;
  block_slice(chunk, blockIdx.x, gridDim.x, lo, hi);
  hi = min(hi, real);
  const T* p = in + (int64_t)c * chunk;
  float mn = FLT_MAX, mx = -FLT_MAX;
  if (vec) {
    // whole 16-byte vectors (consecutive lanes on consecutive vectors), then a scalar tail
    // when `real` cuts a vector
    constexpr int VE = mmdev::Vec16<T>::VE;
    const int64_t full_hi = lo + ((hi > lo ? hi - lo : 0) / VE) * VE;
#pragma unroll 4
    for (int64_t i = lo / VE + threadIdx.x; i < full_hi / VE; i += kThreads) {
      float v[VE];
      mmdev::load_vec(p, i, v);
#pragma unroll
      for (int k = 0; k < VE; ++k) {
        mn = fminf(mn, v[k]);
        mx = fmaxf(mx, v[k]);
      }
    }
    for (int64_t i = full_hi + threadIdx.x; i < hi; i += kThreads) {
      float v = mmdev::to_f(p[i]);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      float v = mmdev::to_f(p[i]);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = make_float2(mn, mx);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    quantise_kernel(const T* __restrict__ in, int64_t chunk, int first_chunk, const float2* __restrict__ partial,
                    int n_partial, uint8_t* __restrict__ out, size_t chunk_offset, bool vec) {
  const int c = first_chunk + blockIdx.y;
  // fold the partials of this chunk
  float mn = FLT_MAX, mx = -FLT_MAX;
  for (int i = threadIdx.x; i < n_partial; i += kThreads) {
    float2 pm = partial[(int64_t)blockIdx.y * n_partial + i];
    mn = fminf(mn, pm.x);
    mx = fmaxf(mx, pm.y);
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (mn > mx) mn = mx = 0.f;  // chunk without real elements
  uint8_t* base = out + (size_t)c * chunk_offset;
  // round through the storage dtype so both sides build the same grid
  const float mn_r = mmdev::to_f(mmdev::from_f<T>(mn));
  const float mx_r = mmdev::to_f(mmdev::from_f<T>(mx));
  if (blockIdx.x == 0 && threadIdx.x == 0) mmdev::store_header<T>(base, mn, mx);
  const mmdev::Grid g = mmdev::make_grid(mn_r, mx_r);
  int64_t lo, hi;
  block_slice(chunk, blockIdx.x, gridDim.x, lo, hi);
  const T* p = in + (int64_t)c * chunk;
  uint8_t* q = base + kCompressHeaderBytes;
  if (vec) {
    constexpr int VE = mmdev::Vec16<T>::VE;
    constexpr int U = 4;
    const int64_t vhi = hi / VE;
    for (int64_t i0 = lo / VE + threadIdx.x; i0 < vhi; i0 += (int64_t)U * kThreads) {
      float v[U][VE];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * kThreads < vhi) mmdev::load_vec(p, i0 + u * kThreads, v[u]);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * kThreads < vhi) mmdev::store_qword(q, i0 + u * kThreads, mmdev::pack_qvec(v[u], g));
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) q[i] = mmdev::quantise(mmdev::to_f(p[i]), g);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    dequantise_kernel(const uint8_t* __restrict__ in, size_t chunk_offset, int64_t chunk, T* __restrict__ out,
                      bool vec) {
  const int c = blockIdx.y;
  const uint8_t* base = in + (size_t)c * chunk_offset;
  float mn, mx;
  mmdev::load_header<T>(base, mn, mx);
  const mmdev::Grid g = mmdev::make_grid(mn, mx);
  int64_t lo, hi;
  block_slice(chunk, blockIdx.x, gridDim.x, lo, hi);
  const uint8_t* q = base + kCompressHeaderBytes;
  T* o = out + (int64_t)c * chunk;
  if (vec) {
    constexpr int VE = mmdev::Vec16<T>::VE;
    __shared__ float s_lut[256];
    mmdev::build_dequant_lut<T>(s_lut, g);
    __syncthreads();
#pragma unroll 4
    for (int64_t i = lo / VE + threadIdx.x; i < hi / VE; i += kThreads) {
      float v[VE];
      mmdev::lut_dqvec(q, i, v, s_lut);
      mmdev::store_vec(o, i, v);
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) o[i] = mmdev::from_f<T>(mmdev::dequantise(q[i], g));
  }
}

template <typename T>
void compress_t(const void* in, int64_t num_real, int64_t chunk, int n_chunks, uint8_t* out, size_t out_bytes,
                int target, void* scratch, size_t scratch_bytes, cudaStream_t s) {
  const size_t off = out_bytes / (size_t)n_chunks;
  const int first = target >= 0 ? target : 0;
  const int count = target >= 0 ? 1 : n_chunks;
  const int bpc = blocks_per_chunk(count, chunk);
  BAGUA_CHECK(scratch != nullptr && scratch_bytes >= (size_t)count * bpc * sizeof(float2), MemPool,
              "compress: scratch buffer too small");
  const bool vec = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && (chunk % 16 == 0) && (off % 16 == 0);
  dim3 grid(bpc, count);
  minmax_partial_kernel<T><<<grid, kThreads, 0, s>>>((const T*)in, num_real, chunk, first, (float2*)scratch, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
  quantise_kernel<T><<<grid, kThreads, 0, s>>>((const T*)in, chunk, first, (const float2*)scratch, bpc, out, off, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

template <typename T>
void decompress_t(const uint8_t* in, size_t in_bytes, int64_t chunk, int n_chunks, void* out, cudaStream_t s) {
  const size_t off = in_bytes / (size_t)n_chunks;
  const bool vec = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && (chunk % 16 == 0) && (off % 16 == 0);
  dim3 grid(blocks_per_chunk(n_chunks, chunk), n_chunks);
  dequantise_kernel<T><<<grid, kThreads, 0, s>>>(in, off, chunk, (T*)out, vec);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

size_t compress_scratch_bytes(int n_chunks, int64_t chunk_size) {
  return (size_t)n_chunks * (size_t)blocks_per_chunk(n_chunks, chunk_size) * sizeof(float2);
}

void compress_minmax_u8(const void* in, DType dt, int64_t num_real, int64_t chunk, int n_chunks, uint8_t* out,
                        size_t out_bytes, int target, void* scratch, size_t scratch_bytes, cudaStream_t s) {
  switch (dt) {
    case DType::F32:
      compress_t<float>(in, num_real, chunk, n_chunks, out, out_bytes, target, scratch, scratch_bytes, s);
      return;
    case DType::F16:
      compress_t<__half>(in, num_real, chunk, n_chunks, out, out_bytes, target, scratch, scratch_bytes, s);
      return;
    case DType::BF16:
      compress_t<__nv_bfloat16>(in, num_real, chunk, n_chunks, out, out_bytes, target, scratch, scratch_bytes, s);
      return;
    default: throw BaguaError(ErrorKind::Tensor, std::string("compress: unsupported dtype ") + dtype_name(dt));
  }
}

void decompress_minmax_u8(const uint8_t* in, size_t in_bytes, int64_t chunk, int n_chunks, void* out, DType dt,
                          cudaStream_t s) {
  switch (dt) {
    case DType::F32: decompress_t<float>(in, in_bytes, chunk, n_chunks, out, s); return;
    case DType::F16: decompress_t<__half>(in, in_bytes, chunk, n_chunks, out, s); return;
    case DType::BF16: decompress_t<__nv_bfloat16>(in, in_bytes, chunk, n_chunks, out, s); return;
    default: throw BaguaError(ErrorKind::Tensor, std::string("decompress: unsupported dtype ") + dtype_name(dt));
  }
}

}  // namespace cuda
}  // namespace kernels
}  // namespace bagua
