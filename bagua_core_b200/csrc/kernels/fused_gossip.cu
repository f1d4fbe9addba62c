// Fused low-precision ring gossip step (one cooperative sm_100a kernel per bucket).
//
// x: local weights after the optimizer step; w / l / r: this rank's replicas of its own,
// its left and its right neighbour's weights.  The step computes
//     d   = x + l/3 + r/3 - 5w/3
//     c   = MinMaxUInt8(d)                       (one chunk, min/max over the whole bucket)
//     send c to both neighbours, receive theirs  (direct peer stores into their staging)
//     l  += Q⁻¹(c_left);  r += Q⁻¹(c_right);  x = w = w + Q⁻¹(c)
// which is what the reference does with 3 addmul kernels, 2 CUB reductions, a compress
// kernel, 4 grouped NCCL send/recv, 3 decompress kernels, 3 add kernels and a memcpy
// (bagua-core-internal/src/comm_ops/decentralized_low_precision_synchronous.rs:23-154).
// Intermediate values are rounded through the tensor dtype where the reference stores them.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>

#include "fused.h"
#include "fused_emu.h"
#include "fused_gossip_body.cuh"
#include "minmax_device.cuh"
#include "peer_sync.cuh"

namespace bagua {
namespace fused {

namespace {

using namespace kernels;
using namespace gossip_bodies;

// one launch per rank
template <typename T>
__global__ void __launch_bounds__(kThreads)
    lp_ring_kernel(const __grid_constant__ ArenaView v, T* __restrict__ x, T* __restrict__ w, T* __restrict__ l,
                   T* __restrict__ r, int64_t n, size_t slot_bytes, size_t scratch_off) {
  lp_ring_body<T>(v, psync::real_launch(), x, w, l, r, n, slot_bytes, scratch_off);
}

// single-GPU emulation: the grids of all ranks in one cooperative launch
template <typename T>
__global__ void __launch_bounds__(kThreads)
    lp_ring_emu_kernel(const EmuRank* __restrict__ ranks, int blocks, int64_t n, size_t slot_bytes,
                       size_t scratch_off) {
  const EmuRank& e = ranks[blockIdx.x / blocks];
  lp_ring_body<T>(e.view, psync::Launch{(int)(blockIdx.x % blocks), blocks}, (T*)e.in, (T*)e.w, (T*)e.l, (T*)e.r, n,
                  slot_bytes, scratch_off);
}

template <typename T>
bool lp_ring_t(PeerArena& arena, void* x, void* w, void* l, void* r, int64_t n, cudaStream_t stream) {
  if (n <= 0) return true;
  if (n % 16 != 0 || ((uintptr_t)x | (uintptr_t)w | (uintptr_t)l | (uintptr_t)r) % 16 != 0) return false;
  const size_t slot = (size_t)n + kHdr;
  int64_t g = (n + (32 << 10) - 1) / (32 << 10);
  int grid = (int)std::max<int64_t>(1, std::min<int64_t>(g, arena.max_coop_blocks()));
  static int coop_limit = 0;
  if (coop_limit == 0) {
    int per_sm = 0, sms = 0, dev = 0;
    BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
    BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lp_ring_kernel<T>, kThreads, 0));
    coop_limit = std::max(1, per_sm * sms);
  }
  grid = std::min(grid, coop_limit);
  const size_t scratch_off = align_up(3 * slot, 256);
  arena.ensure_staging(scratch_off + (size_t)grid * sizeof(float2));
  ArenaView v = arena.next_view(grid, 1);
  T *px = (T*)x, *pw = (T*)w, *pl = (T*)l, *pr = (T*)r;
  int64_t n_arg = n;
  size_t slot_arg = slot, scratch_arg = scratch_off;
  void* args[] = {&v, &px, &pw, &pl, &pr, &n_arg, &slot_arg, &scratch_arg};
  BAGUA_CUDA_CHECK(
      cudaLaunchCooperativeKernel((const void*)lp_ring_kernel<T>, dim3(grid), dim3(kThreads), args, 0, stream));
  arena.count_launch();
  return true;
}

template <typename T>
void emu_lp_ring_t(const EmuRank* dev, int nranks, int blocks, int64_t n, size_t slot_bytes, size_t scratch_off) {
  int per_sm = 0, sms = 0, device = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&device));
  BAGUA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  BAGUA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lp_ring_emu_kernel<T>, kThreads, 0));
  const int grid = nranks * blocks;
  BAGUA_CHECK(grid <= per_sm * sms, Communicator,
              "emulation needs " << grid << " co-resident blocks, the device holds " << per_sm * sms);
  void* args[] = {(void*)&dev, (void*)&blocks, (void*)&n, (void*)&slot_bytes, (void*)&scratch_off};
  BAGUA_CUDA_CHECK(
      cudaLaunchCooperativeKernel((const void*)lp_ring_emu_kernel<T>, dim3(grid), dim3(kThreads), args, 0, 0));
}

}  // namespace

void emu_launch_lp_ring(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, size_t slot_bytes,
                        size_t scratch_off) {
  switch (dt) {
    case DType::F32: emu_lp_ring_t<float>(dev, nranks, blocks, n, slot_bytes, scratch_off); break;
    case DType::F16: emu_lp_ring_t<__half>(dev, nranks, blocks, n, slot_bytes, scratch_off); break;
    case DType::BF16: emu_lp_ring_t<__nv_bfloat16>(dev, nranks, blocks, n, slot_bytes, scratch_off); break;
    default: throw BaguaError(ErrorKind::Tensor, "emulated low-precision ring: unsupported dtype");
  }
}

bool lp_ring(PeerArena& arena, void* x, void* w, void* l, void* r, int64_t n, DType dt, cudaStream_t stream) {
  if (arena.nranks() < 2) return false;
  switch (dt) {
    case DType::F32: return lp_ring_t<float>(arena, x, w, l, r, n, stream);
    case DType::F16: return lp_ring_t<__half>(arena, x, w, l, r, n, stream);
    case DType::BF16: return lp_ring_t<__nv_bfloat16>(arena, x, w, l, r, n, stream);
    default: return false;
  }
}

}  // namespace fused
}  // namespace bagua
