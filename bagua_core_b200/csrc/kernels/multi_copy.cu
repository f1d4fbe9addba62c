// Flatten / unflatten of a staged bucket in ONE launch.
//
// A bucket whose tensors are not address-contiguous is communicated through a flat staging
// buffer (reference: one cudaMemcpyAsync per tensor into the buffer and one per tensor back,
// bagua-core-internal/src/datatypes/mod.rs:1012-1023 and 1048-1059; for a bucket of 400
// tensors that is 800 copies per bucket per step).  Here a table of {tensor address, offset in
// the flat buffer, bytes}, sorted by offset, lives on the device and one kernel moves every
// tensor: the flat byte range is cut into 32 KiB tiles, a CTA finds the first segment of its
// tile by binary search and copies the overlap of every segment with the tile, 16 bytes per
// thread where both sides allow it (4 bytes or single bytes otherwise).
#include <cuda_runtime.h>

#include "kernels_impl.h"

namespace bagua {
namespace kernels {
namespace cuda {

namespace {

constexpr int kMcThreads = 256;
constexpr unsigned long long kTileBytes = 32ull << 10;

// Copies [0, n) bytes; `unit` = 16, 4 or 1: both addresses are multiples of it.
__device__ __forceinline__ void copy_range(char* __restrict__ dst, const char* __restrict__ src,
                                           unsigned long long n, int unit) {
  unsigned long long done = 0;
  if (unit == 16) {
    const unsigned long long nv = n / 16;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    unsigned long long i = threadIdx.x;
    for (; i + 3ull * kMcThreads < nv; i += 4ull * kMcThreads) {
      const uint4 a = s[i], b = s[i + kMcThreads], c = s[i + 2 * kMcThreads], e = s[i + 3 * kMcThreads];
      d[i] = a;
      d[i + kMcThreads] = b;
      d[i + 2 * kMcThreads] = c;
      d[i + 3 * kMcThreads] = e;
    }
    for (; i < nv; i += kMcThreads) d[i] = s[i];
    done = nv * 16;
  } else if (unit == 4) {
    const unsigned long long nw = n / 4;
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    for (unsigned long long i = threadIdx.x; i < nw; i += kMcThreads) d[i] = s[i];
    done = nw * 4;
  }
  for (unsigned long long i = done + threadIdx.x; i < n; i += kMcThreads) dst[i] = src[i];
}

__global__ void __launch_bounds__(kMcThreads)
    multi_copy_kernel(const MultiCopySeg* __restrict__ segs, int nseg, char* flat, unsigned long long total, int gather) {
  const unsigned long long ntiles = (total + kTileBytes - 1) / kTileBytes;
  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const unsigned long long t0 = tile * kTileBytes, t1 = min(t0 + kTileBytes, total);
    // first segment that ends after t0 (segments are sorted by offset and do not overlap)
    int lo = 0, hi = nseg;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (segs[mid].offset + segs[mid].bytes <= t0)
        lo = mid + 1;
      else
        hi = mid;
    }
    for (int k = lo; k < nseg; ++k) {
      const MultiCopySeg sg = segs[k];
      if (sg.offset >= t1) break;
      const unsigned long long a = max(sg.offset, t0), b = min(sg.offset + sg.bytes, t1);
      if (b <= a) continue;
      char* in_flat = flat + a;
      char* in_tensor = reinterpret_cast<char*>(sg.ptr) + (a - sg.offset);
      const unsigned long long both = reinterpret_cast<unsigned long long>(in_flat) |
                                      reinterpret_cast<unsigned long long>(in_tensor);
      const int unit = (both & 15ull) == 0 ? 16 : (both & 3ull) == 0 ? 4 : 1;
      if (gather)
        copy_range(in_flat, in_tensor, b - a, unit);
      else
        copy_range(in_tensor, in_flat, b - a, unit);
    }
  }
}

}  // namespace

void multi_copy(const MultiCopySeg* segs_dev, int nseg, void* flat, size_t total_bytes, bool gather, cudaStream_t s) {
  if (nseg <= 0 || total_bytes == 0) return;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned long long ntiles = (total_bytes + kTileBytes - 1) / kTileBytes;
  const int grid = (int)std::min<unsigned long long>(ntiles, (unsigned long long)sms * 4ull);
  multi_copy_kernel<<<grid, kMcThreads, 0, s>>>(segs_dev, nseg, (char*)flat, (unsigned long long)total_bytes,
                                                gather ? 1 : 0);
  BAGUA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace cuda
}  // namespace kernels
}  // namespace bagua
