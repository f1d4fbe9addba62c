// Communicators: the collective API the ops and the Python layer call.
//
// `SingleCommunicator` = one group of ranks bound to one stream (reference
// `BaguaSingleCommunicator`, bagua-core-internal/src/communicators/mod.rs:19-241).  It
// owns a library transport (NCCL on GPUs, c10d/gloo on host memory) and, on GPUs of one
// NVLink domain, a `PeerArena`: IPC-mapped staging memory and signal words of every
// rank, which the fused sm_100a kernels use to move data with plain peer stores.
//
// `Communicator` adds the two-level form (reference `BaguaCommunicator`,
// communicators/mod.rs:243-428): leader = intranode rank 0 runs
// reduce(intranode) → hook(internode) → broadcast(intranode); workers only take part in
// the reduce and the broadcast.
#pragma once

#include <functional>

#include "../tensor/tensor.h"
#include "transport.h"

namespace bagua {

class PeerArena;

class SingleCommunicator {
 public:
  // unique_id: base64 NCCL id, or "c10d:<group name>" for the host transport
  // (device_id < 0).
  SingleCommunicator(int rank, int nranks, int device_id, uint64_t stream, const std::string& unique_id);
  ~SingleCommunicator();

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  int device_id() const { return device_id_; }
  uint64_t stream() const { return stream_; }
  const char* transport_kind() const { return transport_->kind(); }

  void abort();
  bool check_abort() const { return aborted_.load(std::memory_order_acquire); }

  // Collectives; counts come from num_elements_allocated(), like the reference.
  void allreduce(const RawTensor& send, RawTensor& recv, ReductionOp op);
  // `engine_op`: the call is a bucket's communication (it runs as the fused kernel whenever fused
  // kernels are enabled, whatever set_p2p_collectives says, takes the overlap CTA budget, and
  // first looks at the status record earlier kernels may have left)
  void allreduce_inplace(RawTensor& t, ReductionOp op, bool engine_op = false);
  void broadcast(RawTensor& t, int root);
  void reduce(const RawTensor& send, RawTensor& recv, int dst, ReductionOp op);
  void reduce_inplace(RawTensor& t, int dst, ReductionOp op);
  void send(const RawTensor& t, int peer);
  void recv(RawTensor& t, int peer);
  void alltoall(const RawTensor& send, RawTensor& recv);
  void alltoall_inplace(RawTensor& t);
  void alltoall_v(const RawTensor& send, const std::vector<int64_t>& send_counts,
                  const std::vector<int64_t>& send_displs, RawTensor& recv, const std::vector<int64_t>& recv_counts,
                  const std::vector<int64_t>& recv_displs);
  void allgather(const RawTensor& send, RawTensor& recv);
  void allgather_inplace(RawTensor& t);
  void gather(const RawTensor& send, RawTensor& recv, int dst);
  void gather_inplace(RawTensor& t, int64_t count, int dst);
  void scatter(const RawTensor& send, RawTensor& recv, int src);
  void scatter_inplace(RawTensor& t, int64_t count, int src);
  void reduce_scatter(const RawTensor& send, RawTensor& recv, ReductionOp op);
  void reduce_scatter_inplace(RawTensor& t, ReductionOp op);
  void barrier();
  void group_start() {
    ++group_depth_;
    transport_->group_start();
  }
  void group_end() {
    transport_->group_end();
    if (group_depth_ > 0) --group_depth_;
  }

  // Fused path.  Null when the communicator is on the host, has one rank, was disabled
  // (BAGUA_B200_FUSED=0 or set_fused(false)) or peer mapping failed.
  PeerArena* arena();
  void set_fused(bool on) { fused_enabled_ = on; }
  bool fused_enabled() const { return fused_enabled_; }
  // Throws CommunicatorError if a fused kernel reported a device-side wait that ran out; the
  // communicator is marked aborted and the record is cleared, so the error is raised once and
  // every later use fails with "communicator was aborted".  A plain load of host-mapped memory.
  void check_device_status(bool try_only = false);
  // The same for every live communicator of this process (what `wait_pending_comm_ops` calls).
  static void check_all_device_status();
  // Peer-memory kernels for the collectives above (all-reduce / reduce / reduce-scatter with SUM or
  // AVG, all-gather, all-to-all, gather, scatter, broadcast, barrier) instead of library calls.  Off unless
  // BAGUA_B200_P2P_COLLECTIVES=1 or set_p2p_collectives(true); calls inside a
  // group_start()/group_end() pair and ineligible layouts always take the library path.
  void set_p2p_collectives(bool on) { p2p_collectives_ = on; }
  bool p2p_collectives() const { return p2p_collectives_; }

  Transport& transport() { return *transport_; }

  // Collective over this (intra-node) communicator, once: rank 0 tells the others how many
  // ranks the inter-node communicator it leads has (`mine` is ignored on the other ranks).
  // Later calls return the cached answer without communicating.
  int64_t agree_inter_nranks(int64_t mine);

 private:
  void check_live() const;
  void check_rank(int r, const char* what) const;
  // The arena when this call may run as a peer-memory kernel, else null.
  PeerArena* p2p_arena();
  int rank_, nranks_, device_id_;
  uint64_t stream_;
  std::unique_ptr<Transport> transport_;
  std::atomic<bool> aborted_{false};
  bool fused_enabled_ = true;
  bool p2p_collectives_ = false;
  int group_depth_ = 0;
  bool arena_tried_ = false;
  std::unique_ptr<PeerArena> arena_;
  std::mutex arena_mu_;
  int64_t inter_nranks_ = -1;  // agree_inter_nranks(): not asked yet
};

using SingleCommPtr = std::shared_ptr<SingleCommunicator>;

// RAII ncclGroupStart/End (reference NCCLGroupGuard, communicators/mod.rs:430-453).
class GroupGuard {
 public:
  explicit GroupGuard(SingleCommunicator& c) : c_(c) { c_.group_start(); }
  ~GroupGuard() noexcept(false) { c_.group_end(); }

 private:
  SingleCommunicator& c_;
};

class Communicator {
 public:
  enum class Kind { Single, HierarchicalLeader, HierarchicalWorker };
  // hierarchical=false: `internode` is used alone.  hierarchical=true: `intranode` is
  // required; the rank whose intranode rank is 0 is the leader and needs `internode`.
  static std::shared_ptr<Communicator> create(SingleCommPtr internode, SingleCommPtr intranode, bool hierarchical);

  Kind kind() const { return kind_; }
  // Hierarchical, and the node is the whole job (the inter-node tier has one rank): the
  // intra-node reduce + broadcast pair then runs as one all-reduce on every rank, and the
  // inter-node step runs on every rank over a communicator of one rank (same bits as running
  // it on the leader and broadcasting, one fused kernel instead of two library calls).
  bool single_node() const { return solo_ != nullptr; }
  uint64_t stream() const;
  SingleCommPtr internode() const { return internode_; }
  SingleCommPtr intranode() const { return intranode_; }

  // reference: BaguaCommunicator::execute_communication (communicators/mod.rs:390-427)
  void execute_communication(RawTensor& t, bool intranode_average, bool hierarchical_pre, bool hierarchical_post,
                             const std::function<void(SingleCommunicator&, RawTensor&)>& hook);

 private:
  Kind kind_ = Kind::Single;
  SingleCommPtr internode_, intranode_, solo_;
};

}  // namespace bagua
