// Allocation-free MinMaxUInt8 compression: see capi/bagua_no_alloc.h for the contract.
//
// Same two-launch scheme and the same numerics as the pooled compress path (partial
// min/max per block, then fold + quantise), but the partials live in a fixed array that
// is part of this library's device image instead of a pool allocation.  On the host the
// array's name is only a handle for the runtime; its device address is looked up once
// per device with cudaGetSymbolAddress and passed to the kernels as an ordinary pointer.
#include <cuda_runtime.h>

#include <cfloat>
#include <mutex>
#include <string>

#include "../capi/bagua_no_alloc.h"
#include "kernels.h"
#include "minmax_device.cuh"

namespace {

using namespace bagua::kernels;

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// One copy per GPU that loads the library, held until the process exits.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[BAGUA_NO_ALLOC_SCRATCH_BYTES];

thread_local std::string g_error;
std::mutex g_setup_mu;
void* g_scratch_addr[kMaxDevices] = {};  // device address of the array, per device

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}

inline int blocks_per_chunk(int n_chunks, int64_t chunk) {
  int64_t want = (chunk + 4095) / 4096;
  int64_t cap = std::max<int64_t>(1, (148 * 8) / std::max(1, n_chunks));
  int64_t b = std::min<int64_t>(std::min<int64_t>(want, cap), 1024);
  return (int)std::max<int64_t>(b, 1);
}

__device__ __forceinline__ void block_slice(int64_t chunk, int bx, int nb, int64_t& lo, int64_t& hi) {
  int64_t groups = (chunk + 15) / 16;
  int64_t per = (groups + nb - 1) / nb;
  lo = min((int64_t)bx * per * 16, chunk);
  hi = min(lo + per * 16, chunk);
}

__global__ void __launch_bounds__(kThreads)
    na_minmax_partial(const float* __restrict__ in, int64_t chunk, float2* __restrict__ partial, bool vec) {
  const int c = blockIdx.y;
  int64_t lo, hi;
  block_slice(chunk, blockIdx.x, gridDim.x, lo, hi);
  const float* p = in + (int64_t)c * chunk;
  float mn = FLT_MAX, mx = -FLT_MAX;
  if (vec) {
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float v[16];
      mmdev::load16(p + i, v);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        mn = fminf(mn, v[k]);
        mx = fmaxf(mx, v[k]);
      }
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
      mn = fminf(mn, p[i]);
      mx = fmaxf(mx, p[i]);
    }
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = make_float2(mn, mx);
}

__global__ void __launch_bounds__(kThreads)
    na_quantise(const float* __restrict__ in, int64_t chunk, const float2* __restrict__ partial, uint8_t* __restrict__ out,
                size_t chunk_offset, bool vec) {
  const int c = blockIdx.y;
  float mn = FLT_MAX, mx = -FLT_MAX;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += kThreads) {
    const float2 pm = partial[(int64_t)blockIdx.y * gridDim.x + i];
    mn = fminf(mn, pm.x);
    mx = fmaxf(mx, pm.y);
  }
  mmdev::block_minmax<kThreads>(mn, mx);
  if (mn > mx) mn = mx = 0.f;
  uint8_t* base = out + (size_t)c * chunk_offset;
  if (blockIdx.x == 0 && threadIdx.x == 0) mmdev::store_header<float>(base, mn, mx);
  const mmdev::Grid g = mmdev::make_grid(mn, mx);
  int64_t lo, hi;
  block_slice(chunk, blockIdx.x, gridDim.x, lo, hi);
  const float* p = in + (int64_t)c * chunk;
  uint8_t* q = base + kCompressHeaderBytes;
  if (vec) {
    for (int64_t i = lo + (int64_t)threadIdx.x * 16; i < hi; i += (int64_t)kThreads * 16) {
      float v[16];
      mmdev::load16(p + i, v);
      mmdev::store_q16(q + i, v, g);
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) q[i] = mmdev::quantise(p[i], g);
  }
}

// Device address of the scratch array on the current device; resolved on first use.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(BAGUA_NO_ALLOC_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(BAGUA_NO_ALLOC_ERR_INVALID, "device index out of range");
  std::lock_guard<std::mutex> g(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_no_alloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(BAGUA_NO_ALLOC_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" {

size_t bagua_no_alloc_compressed_size(int64_t num_elements, int n_chunks) {
  if (num_elements <= 0 || n_chunks <= 0 || num_elements % n_chunks != 0) return 0;
  return bagua::align_up((size_t)num_elements, 32) + (size_t)kCompressHeaderBytes * (size_t)n_chunks;
}

const char* bagua_no_alloc_last_error(void) { return g_error.c_str(); }

int bagua_no_alloc_compress_minmax_u8_f32(const float* in, int64_t num_elements, int n_chunks, uint8_t* out,
                                          size_t out_bytes, void* stream) {
  if (!in || !out) return fail(BAGUA_NO_ALLOC_ERR_INVALID, "in and out must be device pointers, got NULL");
  if ((uintptr_t)in % alignof(float) != 0)
    return fail(BAGUA_NO_ALLOC_ERR_INVALID, "in must be aligned to 4 bytes (it is read as float)");
  if (num_elements <= 0 || n_chunks <= 0 || num_elements % n_chunks != 0)
    return fail(BAGUA_NO_ALLOC_ERR_INVALID, "num_elements must be positive and divisible by n_chunks");
  const size_t need = bagua_no_alloc_compressed_size(num_elements, n_chunks);
  if (out_bytes < need)
    return fail(BAGUA_NO_ALLOC_ERR_INVALID,
                "output buffer too small: need " + std::to_string(need) + " bytes, got " + std::to_string(out_bytes));
  const int64_t chunk = num_elements / n_chunks;
  const int bpc = blocks_per_chunk(n_chunks, chunk);
  if ((int64_t)n_chunks * bpc > BAGUA_NO_ALLOC_MAX_PARTIALS)
    return fail(BAGUA_NO_ALLOC_ERR_TOO_LARGE,
                "request needs " + std::to_string((int64_t)n_chunks * bpc) + " partial results, the built-in scratch holds " +
                    std::to_string(BAGUA_NO_ALLOC_MAX_PARTIALS) + " (use fewer chunks or the pooled compress path)");
  void* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  // the layout divides the buffer evenly, exactly like the pooled path
  const size_t off = need / (size_t)n_chunks;
  const bool vec = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && (chunk % 16 == 0) && (off % 16 == 0);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(bpc, n_chunks);
  na_minmax_partial<<<grid, kThreads, 0, s>>>(in, chunk, (float2*)scratch, vec);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    na_quantise<<<grid, kThreads, 0, s>>>(in, chunk, (const float2*)scratch, out, off, vec);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return fail(BAGUA_NO_ALLOC_ERR_CUDA, std::string("kernel launch: ") + cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
