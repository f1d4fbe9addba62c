// Peer arena: the memory every fused communication kernel works through.
//
// Each rank of a communicator allocates (plain cudaMalloc) a staging buffer and a pad
// of 32-bit signal words, exports both as CUDA IPC handles, exchanges the handles with
// an NCCL all-gather on the communicator's own transport, and maps every peer's pair.
// Kernels then move data with ordinary 16-byte stores to peer pointers (NVLink 5 through
// NVSwitch) and synchronise with release/acquire signal words:
//
//   * `done[src]`            – src finished its previous fused op entirely (written by
//                              the last CTA of that op; polled at the start of the next
//                              op, so staging can be reused without a blocking barrier);
//   * `phase[p][src][block]` – block `block` of src finished writing phase p's data into
//                              this rank's staging (block b only ever pairs with block b
//                              of the peers, so no grid-wide sync is needed for data flow);
//   * signal values are the communicator-wide op epoch, which only grows: words are never
//     reset, so there is no reset race.
//
// Every device-side wait is bounded by a deadline; when it runs out the kernel records
// {code, phase, peer, block, epoch} in a host-mapped status record, stops waiting and
// returns.  The host turns a non-zero status into a CommunicatorError and marks the
// communicator aborted; the CUDA context stays usable.
//
// The kernels use ordinary global loads and stores only (no TMA, no cluster features).
// Through staging, remote data is written by its producer into the consumer's memory and
// then read locally; buckets in the symmetric heap are also loaded directly from peers.
#pragma once

#include <cuda_runtime_api.h>

#include "../common.h"
#include "nvls.h"
#include "transport.h"

namespace bagua {

constexpr int kArenaMaxRanks = 8;
// Room for two 512-thread CTAs on each of 148 SMs (the fused kernels stay at or under 64 registers
// per thread, so two are co-resident); the defaults below use far fewer.
constexpr int kArenaMaxBlocks = 320;
constexpr int kArenaPhases = 2;

// Word offsets inside a rank's signal pad.
constexpr int kSigDone = 0;                                   // [kArenaMaxRanks]
constexpr int kSigPhase = 32;                                 // [phases][ranks][blocks]
constexpr int kSigCounter = kSigPhase + kArenaPhases * kArenaMaxRanks * kArenaMaxBlocks;  // local CTA counter
constexpr int kSigPoison = kSigCounter + 1;                   // rank-local: non-zero once a wait ran out or the host aborted
constexpr int kSigGridBar = kSigCounter + 2;                  // 64-bit local grid-barrier counter (2 words, 8 B aligned)
constexpr int kSigWords = kSigGridBar + 6;
static_assert(kSigGridBar % 2 == 0, "the 64-bit grid-barrier counter must sit on an 8-byte boundary");

struct DeviceStatus {
  uint32_t code;    // 0 = ok, 1 = wait on `done`, 2 = wait on a phase flag, 3 = grid barrier, 4 = alltoall_v sizes disagree
  uint32_t phase;
  uint32_t peer;
  uint32_t block;
  uint32_t epoch;
  uint32_t seen;
};

// Passed by value to every fused kernel.
struct ArenaView {
  uint8_t* staging[kArenaMaxRanks];   // this rank's mapping of every rank's staging buffer
  uint32_t* signals[kArenaMaxRanks];  // ... and of every rank's signal pad
  DeviceStatus* status;               // host-mapped
  size_t staging_bytes;
  int rank, nranks;
  uint32_t epoch;                     // this op's epoch (previous op = epoch - 1)
  uint64_t deadline_ns;               // budget of each wait, in ns of %globaltimer
  uint64_t grid_bar_base;             // value of the local grid-barrier counter before this launch
};

class PeerArena {
 public:
  // Collective over `transport` (all ranks construct together).  Throws on failure.
  PeerArena(Transport& transport, int rank, int nranks, int device, cudaStream_t stream);
  ~PeerArena();

  // Collective: make every rank's staging at least `bytes` large.
  void ensure_staging(size_t bytes);
  size_t staging_bytes() const { return staging_bytes_; }
  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  int device() const { return device_; }

  // View for the next fused op; advances the epoch.  `grid` = CTAs the kernel launches,
  // `grid_barriers` = in-kernel grid barriers it executes.
  ArenaView next_view(int grid, int grid_barriers);

  // Max CTAs per fused kernel (BAGUA_B200_COMM_CTAS, default 64, at most kArenaMaxBlocks).
  int max_blocks() const { return max_blocks_; }
  void set_max_blocks(int n) { max_blocks_ = n < 1 ? 1 : (n > kArenaMaxBlocks ? kArenaMaxBlocks : n); }
  void set_max_coop_blocks(int n) { max_coop_blocks_ = n < 1 ? 1 : (n > kArenaMaxBlocks ? kArenaMaxBlocks : n); }
  // Max CTAs of the cooperative kernels (ByteGrad, low-precision ring), which do several
  // HBM passes and quantiser math per element (BAGUA_B200_COOP_CTAS, default 148 = one per SM).
  int max_coop_blocks() const { return max_coop_blocks_; }
  void set_deadline_ms(double ms) { deadline_ns_ = (uint64_t)(ms * 1e6); }
  double deadline_ms() const { return (double)deadline_ns_ / 1e6; }

  // Host view of the status record (all zero when healthy).
  DeviceStatus read_status() const;
  void clear_status();
  // Raises this rank's poison word from the host, on a stream of its own, so that kernels of
  // this rank that are spinning on a peer give up at their next poll (every 32 spins) instead of
  // at their deadline.  Terminal: the word is never cleared, the communicator is finished.
  void poison();
  uint32_t epoch() const { return epoch_; }
  uint64_t fused_launches() const { return launches_; }
  void count_launch() { ++launches_; }

  // ---- symmetric heap ---------------------------------------------------------------
  // Memory that every rank allocates identically (same call sequence, same sizes) and
  // that every peer maps: kernels given a pointer into it can address the same offset
  // on any rank directly, so buckets placed here are reduced in place with no staging
  // copy at all.  Collective when a new slab is needed; memory lives as long as the arena.
  void* sym_alloc(size_t bytes);
  // If [p, p+bytes) lies inside the heap, fills peers[q] with rank q's address of the
  // same offset (peers[rank] == p) and returns true.
  bool sym_translate(const void* p, size_t bytes, void* peers[kArenaMaxRanks]) const;
  size_t sym_bytes_in_use() const { return sym_used_; }
  // If [p, p+bytes) lies inside a slab with an NVSwitch multicast mapping, the multicast
  // address of the same offset (for multimem.ld_reduce / multimem.st); else null.  Slabs get
  // such a mapping when BAGUA_B200_NVLS=1 and the platform supports it (see nvls.h).
  void* sym_multicast(const void* p, size_t bytes) const;
  bool nvls_enabled() const { return nvls_; }

 private:
  void allocate_and_exchange(size_t bytes);
  // Collective: cudaMalloc `bytes` on every rank and map every peer's block.
  void exchange_block(size_t bytes, void** local, void* peers[kArenaMaxRanks]);

  struct Slab {
    char* base[kArenaMaxRanks];  // this rank's mapping of every rank's slab
    size_t bytes;
    size_t used;
    char* mc_base;               // multicast mapping, or null (CUDA-IPC slab)
    MulticastSlab vmm;           // owner of a multicast slab's driver handles
  };
  std::vector<Slab> slabs_;
  size_t sym_used_ = 0;
  mutable std::mutex sym_mu_;

  Transport& transport_;
  int rank_, nranks_, device_;
  cudaStream_t stream_;
  size_t staging_bytes_ = 0;
  void* local_staging_ = nullptr;
  void* local_signals_ = nullptr;
  void release();  // frees and unmaps everything; the destructor, and a constructor that fails
  void* peer_staging_[kArenaMaxRanks] = {};
  void* peer_signals_[kArenaMaxRanks] = {};
  std::vector<void*> retired_;       // superseded local staging buffers, freed at destruction
  std::vector<void*> retired_peer_;  // superseded peer mappings
  DeviceStatus* status_host_ = nullptr;  // 64 pinned, mapped bytes: the record, and at word 15 a constant 1
  DeviceStatus* status_dev_ = nullptr;
  cudaStream_t abort_stream_ = nullptr;  // carries poison(); never blocked by a spinning kernel
  uint32_t epoch_ = 0;
  uint64_t grid_bar_ = 0;
  uint64_t deadline_ns_;
  int max_blocks_;
  int max_coop_blocks_;
  bool nvls_ = false;
  uint64_t launches_ = 0;
};

}  // namespace bagua
