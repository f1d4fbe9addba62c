#include "fused.h"
namespace bagua { namespace fused {
bool bytegrad(PeerArena&, void*, int64_t, DType, bool, cudaStream_t) { return false; }
bool lp_ring(PeerArena&, void*, void*, void*, void*, int64_t, DType, cudaStream_t) { return false; }
}}
