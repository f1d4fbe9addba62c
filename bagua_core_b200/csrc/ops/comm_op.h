// Communication ops: what a bucket does when the scheduler hands it to the worker.
//
// Reference: trait CommOpTrait and its six implementations
// (bagua-core-internal/src/comm_ops/*.rs).  Every op follows the same frame:
// take the bucket's flat communication tensor on the communicator's stream (waiting on
// the tensors' ready events), run the algorithm through
// `Communicator::execute_communication`, release the tensor.  On a GPU communicator
// with a peer arena the algorithm body is ONE fused sm_100a kernel; otherwise (host
// memory, baseline mode, ineligible layout) it is the reference's sequence of library
// collectives and element-wise kernels.
//
// Unlike the reference, ops do not synchronise the stream per bucket unless
// `EngineConfig::sync_per_bucket` is set (baseline mode); buckets pipeline on the stream.
#pragma once

#include "../comm/communicator.h"
#include "../runtime/stats.h"
#include "../tensor/tensor.h"

namespace bagua {

struct EngineConfig {
  // Reference-faithful host behaviour: cudaStreamSynchronize after every bucket.
  bool sync_per_bucket = false;
  static EngineConfig& global();
};

class CommOp {
 public:
  virtual ~CommOp() = default;
  virtual void execute_background_communication(const BucketPtr& bucket) = 0;
  virtual std::string describe() const = 0;
  // State worth checkpointing (e.g. the gossip step counter); empty for stateless ops.
  virtual std::vector<std::pair<std::string, int64_t>> state() const { return {}; }
  virtual void load_state(const std::vector<std::pair<std::string, int64_t>>&) {}
};

enum class PeerSelectionMode { All, ShiftOne, Ring };
PeerSelectionMode parse_peer_selection_mode(const std::string& s);

// shift_one pairing (reference: decentralized_full_precision_synchronous.rs:66-76):
// the lower half of the ranks pairs with the upper half, rotating by one every step.
int shift_one_peer(int rank, int nranks, int64_t step);

std::shared_ptr<CommOp> make_centralized_full_precision_op(std::shared_ptr<Communicator> comm, bool average,
                                                           bool scattergather);
std::shared_ptr<CommOp> make_centralized_low_precision_op(std::shared_ptr<Communicator> comm, bool average,
                                                          const std::string& compression);
std::shared_ptr<CommOp> make_decentralized_full_precision_op(std::shared_ptr<Communicator> comm,
                                                             PeerSelectionMode mode, TensorPtr peer_weight);
std::shared_ptr<CommOp> make_decentralized_low_precision_op(std::shared_ptr<Communicator> comm,
                                                            PeerSelectionMode mode, const std::string& compression,
                                                            TensorPtr weight, TensorPtr left_peer_weight,
                                                            TensorPtr right_peer_weight);
std::shared_ptr<CommOp> make_decentralized_async_op(std::shared_ptr<Communicator> comm, PeerSelectionMode mode,
                                                    uint64_t torch_stream);
// `call(bucket_name)` runs on the worker thread; the bindings wrap a Python callable.
std::shared_ptr<CommOp> make_callback_op(std::function<void(const std::string&)> call, std::string label);

}  // namespace bagua
