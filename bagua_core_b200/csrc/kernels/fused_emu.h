// Single-GPU emulation of the fused communication kernels.
//
// Kernels whose blocks wait on blocks of other ranks cannot be tested on one GPU by
// launching one kernel per rank (nothing guarantees that separate launches run at the
// same time).  The emulation instead hosts the grids of all N ranks side by side in ONE
// cooperative launch: block index / G selects the virtual rank, block index % G is the
// block's position inside that rank's grid, and every virtual rank gets its own staging
// buffer, signal pad and ArenaView on the same device.  The device code that runs is the
// same `*_body` function the real kernels call; only the `Launch` position differs.
// Used by the GPU tests on machines with fewer GPUs than ranks and for profiling a fused
// kernel from a single process.
#pragma once

#include <cuda_runtime_api.h>

#include <vector>

#include "../comm/arena.h"
#include "../common.h"

namespace bagua {
namespace fused {

struct EmuRank {
  ArenaView view;
  const void* in;   // all-reduce / pair-average input, ByteGrad bucket, lp-ring x
  void* out;        // all-reduce / pair-average output
  void* w;          // lp-ring replicas
  void* l;
  void* r;
  const void* sym_in[kArenaMaxRanks];  // symmetric all-reduce: every rank's input / output
  void* sym_out[kArenaMaxRanks];
  int peer;         // pair-average partner
};

enum class EmuAllreduceMode { OneShot = 1, TwoShot = 2, Symmetric = 3, SymmetricTma = 4 };
enum class EmuCollective {
  AllGather = 1,
  AllToAll = 2,
  ReduceScatter = 3,
  BroadcastDirect = 4,
  BroadcastTwoPhase = 5,
  Barrier = 6,
  Scatter = 7,
  Gather = 8,
  ReduceDirect = 9,
  ReduceTwoPhase = 10
};

class EmulatedArena {
 public:
  EmulatedArena(int nranks, int device, size_t staging_bytes);
  ~EmulatedArena();
  EmulatedArena(const EmulatedArena&) = delete;

  int nranks() const { return nranks_; }
  // Pointers are per rank (index = rank), all on this arena's device.  Calls are
  // synchronous: they return after the kernel finished, and throw CommunicatorError if a
  // device-side wait ran out.
  void allreduce(const std::vector<const void*>& in, const std::vector<void*>& out, int64_t n, DType dt, float scale,
                 EmuAllreduceMode mode, int blocks);
  void bytegrad(const std::vector<void*>& buckets, int64_t n, DType dt, bool average, int blocks);
  // symmetric = true: partners load each other's input directly instead of going through staging
  void pair_average(const std::vector<const void*>& in, const std::vector<void*>& out, int64_t n, DType dt,
                    const std::vector<int>& peers, int blocks, bool symmetric = false);
  void lp_ring(const std::vector<void*>& x, const std::vector<void*>& w, const std::vector<void*>& l,
               const std::vector<void*>& r, int64_t n, DType dt, int blocks);
  // The communicator's own collectives.  AllGather / AllToAll / ReduceScatter: `chunk_bytes`
  // per chunk, in[r] / out[r] per rank (in-place forms allowed); `symmetric` selects the
  // variants that store into (exchange) or load from (reduce-scatter) the peers' buffers
  // directly.  Broadcast*: `out[r]` is rank r's buffer of `chunk_bytes`, `root` the source.
  // Scatter: in[r] holds N chunks (read on the root), out[r] one.  Gather: in[r] one chunk,
  // out[r] N chunks (written on the root).  Reduce*: in[r] and out[r] of `chunk_bytes`, the
  // sum lands in out[root].  Barrier: no buffers.
  void collective(EmuCollective kind, const std::vector<const void*>& in, const std::vector<void*>& out,
                  size_t chunk_bytes, DType dt, float scale, int root, bool symmetric, int blocks);
  // All-to-all with per-pair sizes: rank s sends bytes[s * N + d] bytes to rank d; segments are
  // packed back to back in in[s] (in destination order) and in out[d] (in source order).
  void alltoall_v(const std::vector<const void*>& in, const std::vector<void*>& out,
                  const std::vector<int64_t>& bytes, int blocks);
  void set_deadline_ms(double ms) { deadline_ns_ = (uint64_t)(ms * 1e6); }
  uint32_t epoch() const { return epoch_; }

 private:
  // Fills one EmuRank per rank with the view of the next op; returns the device copy.
  EmuRank* prepare(std::vector<EmuRank>& host, int blocks, int grid_barriers, size_t staging_needed);
  void finish(const char* what);

  int nranks_, device_;
  size_t staging_bytes_;
  std::vector<void*> staging_, signals_;
  DeviceStatus* status_host_ = nullptr;
  DeviceStatus* status_dev_ = nullptr;
  EmuRank* dev_args_ = nullptr;
  uint32_t epoch_ = 0;
  uint64_t grid_bar_ = 0;
  uint64_t deadline_ns_ = 5000000000ull;
};

// Launchers defined next to the kernels they start (cooperative, nranks*blocks CTAs).
void emu_launch_allreduce(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale,
                          EmuAllreduceMode mode, int64_t aux_vecs);
// The bulk-copy (TMA) variant of the symmetric all-reduce; 2, 4 or 8 ranks.
void emu_launch_allreduce_tma(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale);
void emu_launch_pair_average(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, bool symmetric);
// aux: bit 0 = symmetric variant, bit 1 = local chunk already in place (exchange);
// the root rank for the broadcasts; root | in_place << 8 for scatter, gather and reduce.
void emu_launch_collective(const EmuRank* dev, int nranks, int blocks, EmuCollective kind, int64_t cvec, DType dt,
                           int aux, float scale);
// `segments`: device array of one fused::collectives::VSegments per rank.
void emu_launch_alltoall_v(const EmuRank* dev, const void* segments, int nranks, int blocks);
void emu_launch_bytegrad(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, float scale,
                         size_t slot_bytes, size_t scratch_off);
void emu_launch_lp_ring(const EmuRank* dev, int nranks, int blocks, int64_t n, DType dt, size_t slot_bytes,
                        size_t scratch_off);

}  // namespace fused
}  // namespace bagua
