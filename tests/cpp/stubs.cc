// Link-time stand-ins for the parts of the engine the host-runtime stress test never calls
// (communicators, fused kernels, CUDA launchers).  Each aborts if it is reached.
#include <cstdlib>

#include "comm/arena.h"
#include "comm/communicator.h"
#include "kernels/fused.h"
#include "kernels/kernels_impl.h"

#define UNREACHABLE() std::abort()

namespace bagua {
PeerArena* SingleCommunicator::arena() { UNREACHABLE(); }
void SingleCommunicator::check_device_status(bool) { UNREACHABLE(); }
void SingleCommunicator::check_all_device_status() {}  // host-only backends never reach it; harmless if they do
void SingleCommunicator::allreduce(const RawTensor&, RawTensor&, ReductionOp) { UNREACHABLE(); }
void SingleCommunicator::allreduce_inplace(RawTensor&, ReductionOp, bool) { UNREACHABLE(); }
void SingleCommunicator::alltoall_inplace(RawTensor&) { UNREACHABLE(); }
void SingleCommunicator::allgather_inplace(RawTensor&) { UNREACHABLE(); }
void SingleCommunicator::send(const RawTensor&, int) { UNREACHABLE(); }
void SingleCommunicator::recv(RawTensor&, int) { UNREACHABLE(); }
uint64_t Communicator::stream() const { UNREACHABLE(); }
void Communicator::execute_communication(RawTensor&, bool, bool, bool,
                                         const std::function<void(SingleCommunicator&, RawTensor&)>&) {
  UNREACHABLE();
}
namespace fused {
bool allreduce(PeerArena&, const void*, void*, int64_t, DType, float, cudaStream_t, bool) { UNREACHABLE(); }
bool bytegrad(PeerArena&, void*, int64_t, DType, bool, cudaStream_t, bool) { UNREACHABLE(); }
bool pair_average(PeerArena&, const void*, void*, int64_t, DType, int, cudaStream_t) { UNREACHABLE(); }
void debug_occupy(void*, size_t, int, int, double, int, cudaStream_t) { UNREACHABLE(); }
bool lp_ring(PeerArena&, void*, void*, void*, void*, int64_t, DType, cudaStream_t) { UNREACHABLE(); }
}  // namespace fused
namespace kernels {
namespace cuda {
void divide_inplace(void*, DType, int64_t, float, cudaStream_t) { UNREACHABLE(); }
void add_inplace(void*, const void*, DType, int64_t, cudaStream_t) { UNREACHABLE(); }
void subtract_inplace(void*, const void*, DType, int64_t, cudaStream_t) { UNREACHABLE(); }
void addmul_inplace(void*, const void*, float, DType, int64_t, cudaStream_t) { UNREACHABLE(); }
void average_inplace(void*, const void*, DType, int64_t, cudaStream_t) { UNREACHABLE(); }
void async_model_average(float*, const float*, const float*, float, int64_t, cudaStream_t) { UNREACHABLE(); }
void copy_bytes(void*, const void*, size_t, cudaStream_t) { UNREACHABLE(); }
void multi_copy(const MultiCopySeg*, int, void*, size_t, bool, cudaStream_t) { UNREACHABLE(); }
void reduce_chunk_inplace(void*, DType, int64_t, int, int, bool, cudaStream_t) { UNREACHABLE(); }
size_t compress_scratch_bytes(int, int64_t) { return 0; }
void compress_minmax_u8(const void*, DType, int64_t, int64_t, int, uint8_t*, size_t, int, void*, size_t, cudaStream_t) {
  UNREACHABLE();
}
void decompress_minmax_u8(const uint8_t*, size_t, int64_t, int, void*, DType, cudaStream_t) { UNREACHABLE(); }
void sgd_momentum_flat(float*, const float*, float*, int64_t, float, float, float, float, bool, bool, cudaStream_t) {
  UNREACHABLE();
}
void sgd_momentum_flat_shadow(float*, const float*, float*, void*, int64_t, float, float, float, float, bool, bool,
                              cudaStream_t) {
  UNREACHABLE();
}
}  // namespace cuda
}  // namespace kernels
}  // namespace bagua
