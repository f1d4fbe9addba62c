// Fused ByteGrad: the whole MinMaxUInt8-compressed all-reduce of one bucket in ONE
// cooperative sm_100a kernel, exchanging compressed chunks by direct peer stores.
//
// Phases (block b of every rank owns the same 16-element groups of every chunk):
//   P1  partial min/max of my slice of each of the N chunks            → local scratch
//       ── grid barrier ──
//   P2  fold partials → grid per chunk; quantise my slice of chunk c and store it, with
//       the {min,max} header, straight into slot[me] of rank c's staging; signal c
//   P3  wait for the N-1 signals; dequantise the N slots of my chunk, sum in rank order
//       (fp32), scale, round to the tensor dtype into the bucket; partial min/max
//       ── grid barrier ──
//   P4  fold → grid; quantise the reduced slice once and store it into slot[me] of every
//       rank's all-gather area; signal everyone
//   P5  wait; dequantise slice b of all N chunks into the bucket
//
// HBM traffic ≈ 2 reads + 1 write of the bucket plus the 1-byte payloads; wire traffic is
// 2(N-1)/N · (S/4 + headers) per GPU.  The reference runs ≥ 40 launches and two NCCL
// collectives per bucket for the same result
// (bagua-core-internal/src/comm_ops/centralized_low_precision_synchronous.rs:16-73).
// Numerics follow the reference: values are rounded through the tensor dtype after every
// dequantise and after the reduction, headers are stored in the tensor dtype.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "fused.h"
#include "fused_emu.h"
#include "fused_bytegrad_body.cuh"
#include "minmax_device.cuh"
#include "peer_sync.cuh"

namespace bagua {
namespace fused {

namespace {

using namespace kernels;
using namespace bytegrad_bodies;

// one launch per rank
template <typename T>
__global__ void __launch_bounds__(kThreads)
    bytegrad_kernel(const __grid_constant__ ArenaView v, T* __restrict__ x, int64_t chunk, size_t slot_bytes,
                    size_t scratch_off, float scale, int pipelined) {
  bytegrad_body<T>(v, psync::real_launch(), x, chunk, slot_bytes, scratch_off, scale, pipelined != 0);
}

// Whether the reduced chunks travel back one destination at a time (see bytegrad_body): for chunks of
// at least BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK bytes; unset or negative = never (the default until
// the variant has been timed).  Read at every call, and the same on every rank, like all environment knobs.
bool pipelined_for(size_t chunk_bytes) {
  const long min_chunk = env_long("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", -1);
  return min_chunk >= 0 && chunk_bytes >= (size_t)min_chunk;
}

// single-GPU emulation: the grids of all ranks in one cooperative launch
template <typename T>
__global__ void __launch_bounds__(kThreads)
    bytegrad_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int64_t chunk, size_t slot_bytes,
                        size_t scratch_off, float scale, int pipelined) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  bytegrad_body<T>(e.view, psync::Launch{(int)(blockIdx.x % blocks), blocks}, (T*)e.in, chunk, slot_bytes, scratch_off,
                   scale, pipelined != 0);
}

template <typename T>
bool bytegrad_t(PeerArena& arena, void* bucket, int64_t n, bool average, cudaStream_t stream, bool overlapped) {
  const int N = arena.nranks();
  if (n <= 0) return true;
  if (n % ((int64_t)16 * N) != 0 || (uintptr_t)bucket % 16 != 0) return false;
  const int64_t chunk = n / N;
  if ((chunk * (int64_t)sizeof(T)) % 16 != 0) return false;
  const size_t slot = (size_t)chunk + kHdr;
  // one CTA per 32 Ki elements of the bucket, up to the arena's limit for cooperative
  // kernels (one per SM by default: several HBM passes plus quantiser math per element)
  int64_t g = (n + (32 << 10) - 1) / (32 << 10);
  // A cooperative launch starts only when all of its CTAs fit on the GPU at once.  With one CTA
  // per SM that means an idle GPU: the bucket then waits for the running backward kernels to
  // drain and the kernels queued behind it wait for the bucket.  A bucket reduced during
  // backward therefore takes the (smaller) overlap budget, which the GPU frees up quickly.
  int64_t cap = arena.max_coop_blocks();
  if (overlapped) cap = std::min<int64_t>(cap, std::max<long>(Tuning::global().coop_overlap_ctas.load(), 1));
  int grid = (int)std::max<int64_t>(1, std::min<int64_t>(g, cap));
  static int coop_limit = 0;
  if (coop_limit == 0) {
    int per_sm = 0, sms = 0, dev = 0;
    BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
    BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bytegrad_kernel<T>, kThreads, 0));
    coop_limit = std::max(1, per_sm * sms);
  }
  grid = std::min(grid, coop_limit);
  const size_t scratch_off = align_up(2 * (size_t)N * slot, 256);
  arena.ensure_staging(scratch_off + (size_t)(N + 1) * grid * sizeof(float2));
  ArenaView v = arena.next_view(grid, 2);
  T* x = (T*)bucket;
  int64_t chunk_arg = chunk;
  size_t slot_arg = slot, scratch_arg = scratch_off;
  float scale = average ? 1.0f / (float)N : 1.0f;
  int pipelined = pipelined_for((size_t)chunk * sizeof(T)) ? 1 : 0;
  void* args[] = {&v, &x, &chunk_arg, &slot_arg, &scratch_arg, &scale, &pipelined};
  BAGUA_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)bytegrad_kernel<T>, dim3(grid), dim3(kThreads), args, 0,
                                               stream));
  arena.count_launch();
  return true;
}

template <typename T>
void emu_bytegrad_t(const EmuRank* dev, int nranks, int blocks, int64_t n, float scale, size_t slot_bytes,
                    size_t scratch_off) {
  int per_sm = 0, sms = 0, device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bytegrad_emu_kernel<T>, kThreads, 0));
  const int grid = nranks * blocks;
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  int64_t chunk = n / nranks;
  int pipelined = pipelined_for((size_t)chunk * sizeof(T)) ? 1 : 0;
  void* args[] = {(void*)&dev, (void*)&blocks, (void*)&chunk, (void*)&slot_bytes, (void*)&scratch_off, (void*)&scale,
                  (void*)&pipelined};
  BAGUA_CUDA_CHECK(
      cudaLaunchCooperativeKernel((const void*)bytegrad_emu_kernel<T>, dim3(grid), dim3(kThreads), args, 0, 0));
}

}  // namespace

void emu_launch_bytegrad(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale,
                         size_t slot_bytes, size_t scratch_off) {
  switch (dt) {
    case DType::F32: emu_bytegrad_t<float>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    case DType::F16: emu_bytegrad_t<__half>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    case DType::BF16: emu_bytegrad_t<__nv_bfloat16>(dev, nranks, blocks, n, scale, slot_bytes, scratch_off); break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated ByteGrad: unsupported dtype");
  }
}

bool bytegrad(PeerArena& arena, void* bucket, int64_t n, DType dt, bool average, cudaStream_t stream,
              bool overlapped) {
  switch (dt) {
    case DType::F32: return bytegrad_t<float>(arena, bucket, n, average, stream, overlapped);
    case DType::F16: return bytegrad_t<__half>(arena, bucket, n, average, stream, overlapped);
    case DType::BF16: return bytegrad_t<__nv_bfloat16>(arena, bucket, n, average, stream, overlapped);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
