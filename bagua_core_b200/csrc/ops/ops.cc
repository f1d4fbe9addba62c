// The six communication ops.  Each has a fused body (one sm_100a kernel over the peer
// arena) and a library body that replays the reference's call sequence; the library
// body is also the CPU backend and the measured baseline.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "../comm/arena.h"
#include "../kernels/fused.h"
#include "../runtime/timeline.h"
#include "comm_op.h"

namespace bagua {

EngineConfig& EngineConfig::global() {
  static EngineConfig c = [] {
    EngineConfig e;
    e.sync_per_bucket = env_long("BAGUA_B200_SYNC_PER_BUCKET", 0) != 0;
    return e;
  }();
  return c;
}
EngineStats& EngineStats::global() {
  static EngineStats s;
  return s;
}

PeerSelectionMode parse_peer_selection_mode(const std::string& s) {
  if (s == "all") return PeerSelectionMode::All;
  if (s == "shift_one") return PeerSelectionMode::ShiftOne;
  if (s == "ring") return PeerSelectionMode::Ring;
  throw BaguaError(ErrorKind::Bucket, "unsupported peer_selection_mode `" + s + "`");
}

int shift_one_peer(int rank, int nranks, int64_t step) {
  const int64_t r = rank, n = nranks, h = n / 2;
  if (r < h) return (int)(((step + r) % ((n + 1) / 2)) + h);
  int64_t v = (r - h - step) % h;
  if (v < 0) v += h;
  return (int)v;
}

namespace {

// Arena of the communicator the hook runs on, or null when the fused path is off.  Before the
// next fused kernel is launched on an arena, the status record its earlier kernels may have
// left is read (host-mapped memory, a plain load): a wait that ran out makes this op fail, the
// failure reaches the caller of `wait_pending_comm_ops`, and no further kernel is started
// on a communicator that is aborted (its poison word would make each give up at once and
// leave its bucket unreduced).
PeerArena* fused_arena(SingleCommunicator& c, const RawTensor& t) {
  if (t.device_id() < 0 || c.nranks() < 2 || !c.fused_enabled()) return nullptr;
  PeerArena* a = c.arena();
  if (!a) return nullptr;
  c.check_device_status();
  if (c.check_abort()) throw BaguaError(ErrorKind::Communicator, "communicator was aborted");
  return a;
}

void note_fused() { EngineStats::global().fused_launches++; }
void note_fallback() { EngineStats::global().library_fallbacks++; }

struct OpFrame {
  // Common prologue/epilogue of an op: lock, stream, communication tensor, release.
  OpFrame(const BucketPtr& bucket, Communicator& comm, bool force_copy, bool no_copy_back)
      : lock(bucket->exec_mutex()), stream(comm.stream()) {
    ct = bucket->get_communication_tensor(stream, force_copy, no_copy_back);
    if (ct.staged) EngineStats::global().staged_copies++;
    EngineStats::global().bytes_communicated += ct.raw->bytes_allocated();
    gpu = ct.raw->device_id() >= 0;
    // device time line: the span opens after the waits on the tensors' ready events
    if (gpu) ticket = BucketTimeline::instance().begin(bucket->name(), ct.raw->bytes_allocated(), (cudaStream_t)stream);
  }
  void finish() {
    if (ticket) BucketTimeline::instance().end(ticket, (cudaStream_t)stream);
    const bool sync = EngineConfig::global().sync_per_bucket;
    ct.finish(sync);
    // after a stream synchronisation the status record is final for this bucket
    if (gpu && sync) SingleCommunicator::check_all_device_status();
  }
  std::unique_lock<std::mutex> lock;
  uint64_t stream;
  CommunicationTensor ct;
  bool gpu = false;
  uint64_t ticket = 0;
};

// ---------------------------------------------------------------------------------
// O1: centralized, full precision, synchronous (gradient all-reduce)
// ---------------------------------------------------------------------------------
class CentralizedFullPrecisionSynchronous : public CommOp {
 public:
  CentralizedFullPrecisionSynchronous(std::shared_ptr<Communicator> c, bool average, bool scattergather)
      : comm_(std::move(c)), average_(average), scattergather_(scattergather) {}

  void execute_background_communication(const BucketPtr& bucket) override {
    OpFrame f(bucket, *comm_, false, false);
    comm_->execute_communication(*f.ct.raw, average_, true, true, [&](SingleCommunicator& c, RawTensor& t) {
      if (c.nranks() == 1) {
        // Sum or mean over one rank: nothing to do.  With BAGUA_B200_PROBE_OCCUPY="ctas,threads,us_per_mb,mode"
        // a stand-in kernel takes the place of the bucket's communication (same stream, same moment, a
        // duration in proportion to the bucket's size), which shows on ONE GPU what a communication
        // kernel of that shape costs the backward pass it overlaps (benchmarks/interference_probe.py).
        static const std::string probe = [] {
          const char* e = std::getenv("BAGUA_B200_PROBE_OCCUPY");
          return std::string(e ? e : "");
        }();
        if (!probe.empty() && t.device_id() >= 0) {
          int ctas = 0, threads = 0, mode = 0;
          double us_per_mb = 0;
          if (std::sscanf(probe.c_str(), "%d,%d,%lf,%d", &ctas, &threads, &us_per_mb, &mode) == 4) {
            const double mb = (double)t.bytes_allocated() / (1 << 20);
            fused::debug_occupy(t.data_ptr(), t.bytes_allocated(), ctas, threads, 15.0 + us_per_mb * mb, mode,
                                (cudaStream_t)c.stream());
          }
        }
        return;
      }
      if (PeerArena* a = fused_arena(c, t)) {
        const float scale = average_ ? 1.0f / (float)c.nranks() : 1.0f;
        if (fused::allreduce(*a, t.data_ptr(), t.data_ptr(), t.num_elements_allocated(), t.dtype(), scale,
                             (cudaStream_t)c.stream(), /*overlapped=*/true)) {
          note_fused();
          return;
        }
        note_fallback();
      }
      if (scattergather_) {
        c.alltoall_inplace(t);
        if (average_)
          tensor_ops::reduce_mean_inplace(t, c.nranks(), c.rank(), c.stream());
        else
          tensor_ops::reduce_sum_inplace(t, c.nranks(), c.rank(), c.stream());
        c.allgather_inplace(t);
      } else {
        c.allreduce_inplace(t, average_ ? ReductionOp::AVG : ReductionOp::SUM);
      }
    });
    f.finish();
  }
  std::string describe() const override {
    std::ostringstream o;
    o << "CentralizedFullPrecisionSynchronous{average=" << average_ << ", scattergather=" << scattergather_ << "}";
    return o.str();
  }

 private:
  std::shared_ptr<Communicator> comm_;
  bool average_, scattergather_;
};

// ---------------------------------------------------------------------------------
// O2: centralized, low precision, synchronous (ByteGrad)
// ---------------------------------------------------------------------------------
class CentralizedLowPrecisionSynchronous : public CommOp {
 public:
  CentralizedLowPrecisionSynchronous(std::shared_ptr<Communicator> c, bool average, std::string method)
      : comm_(std::move(c)), average_(average), method_(std::move(method)) {
    BAGUA_CHECK(method_ == "MinMaxUInt8", Bucket, "unsupported compression `" << method_ << "`");
  }

  void execute_background_communication(const BucketPtr& bucket) override {
    OpFrame f(bucket, *comm_, false, false);
    comm_->execute_communication(*f.ct.raw, average_, true, true, [&](SingleCommunicator& c, RawTensor& t) {
      if (PeerArena* a = fused_arena(c, t)) {
        if (fused::bytegrad(*a, t.data_ptr(), t.num_elements_allocated(), t.dtype(), average_,
                            (cudaStream_t)c.stream(), /*overlapped=*/true)) {
          note_fused();
          return;
        }
        note_fallback();
      }
      const int n = c.nranks();
      auto compressed = tensor_ops::compress(t, method_, n, c.stream(), -1);
      c.alltoall_inplace(*compressed);
      tensor_ops::decompress_from(t, method_, n, *compressed, c.stream());
      if (average_)
        tensor_ops::reduce_mean_inplace(t, n, c.rank(), c.stream());
      else
        tensor_ops::reduce_sum_inplace(t, n, c.rank(), c.stream());
      auto recompressed = tensor_ops::compress(t, method_, n, c.stream(), c.rank());
      c.allgather_inplace(*recompressed);
      tensor_ops::decompress_from(t, method_, n, *recompressed, c.stream());
    });
    f.finish();
  }
  std::string describe() const override {
    std::ostringstream o;
    o << "CentralizedLowPrecisionSynchronous{average=" << average_ << ", compression=" << method_ << "}";
    return o.str();
  }

 private:
  std::shared_ptr<Communicator> comm_;
  bool average_;
  std::string method_;
};

// ---------------------------------------------------------------------------------
// O3: decentralized, full precision, synchronous (gossip)
// ---------------------------------------------------------------------------------
class DecentralizedFullPrecisionSynchronous : public CommOp {
 public:
  DecentralizedFullPrecisionSynchronous(std::shared_ptr<Communicator> c, PeerSelectionMode mode, TensorPtr peer_weight)
      : comm_(std::move(c)), mode_(mode), peer_weight_(std::move(peer_weight)) {
    BAGUA_CHECK(mode_ == PeerSelectionMode::All || mode_ == PeerSelectionMode::ShiftOne, Bucket,
                "decentralized synchronous op supports peer_selection_mode all / shift_one");
  }

  void execute_background_communication(const BucketPtr& bucket) override {
    const bool leader = comm_->kind() == Communicator::Kind::HierarchicalLeader;
    OpFrame f(bucket, *comm_, leader, leader);
    auto peer = peer_weight_->raw();
    const int64_t step = step_.load();
    // The averaged weights are left in `peer_weight`; the caller copies them back.
    comm_->execute_communication(*f.ct.raw, true, true, false, [&](SingleCommunicator& c, RawTensor& t) {
      BAGUA_CHECK(peer->num_elements_allocated() == t.num_elements_allocated() && peer->dtype() == t.dtype(), Tensor,
                  "peer_weight must have the bucket's size and dtype");
      PeerArena* a = fused_arena(c, t);
      if (mode_ == PeerSelectionMode::All) {
        if (a && fused::allreduce(*a, t.data_ptr(), peer->data_ptr(), t.num_elements_allocated(), t.dtype(),
                                  1.0f / (float)c.nranks(), (cudaStream_t)c.stream())) {
          note_fused();
          return;
        }
        if (a) note_fallback();
        tensor_ops::clone_from(*peer, t, c.stream());
        c.allreduce_inplace(*peer, ReductionOp::AVG);
      } else {
        BAGUA_CHECK(c.nranks() % 2 == 0, Communicator,
                    "you cannot use decentralized algorithm with average_all off when there are odd number of "
                    "ranks, current n_ranks "
                        << c.nranks());
        const int peer_rank = shift_one_peer(c.rank(), c.nranks(), step);
        BAGUA_LOG(Debug, "rank " << c.rank() << " peer_rank " << peer_rank);
        if (a && fused::pair_average(*a, t.data_ptr(), peer->data_ptr(), t.num_elements_allocated(), t.dtype(),
                                     peer_rank, (cudaStream_t)c.stream())) {
          note_fused();
          return;
        }
        if (a) note_fallback();
        {
          GroupGuard g(c);
          c.send(t, peer_rank);
          c.recv(*peer, peer_rank);
        }
        tensor_ops::average_inplace(*peer, t, c.stream());
      }
    });
    f.finish();
    step_++;
  }
  std::string describe() const override {
    std::ostringstream o;
    o << "DecentralizedFullPrecisionSynchronous{peer_selection_mode="
      << (mode_ == PeerSelectionMode::All ? "all" : "shift_one") << ", step=" << step_.load() << "}";
    return o.str();
  }
  std::vector<std::pair<std::string, int64_t>> state() const override { return {{"step", step_.load()}}; }
  void load_state(const std::vector<std::pair<std::string, int64_t>>& s) override {
    for (auto& kv : s)
      if (kv.first == "step") step_ = kv.second;
  }

 private:
  std::shared_ptr<Communicator> comm_;
  PeerSelectionMode mode_;
  TensorPtr peer_weight_;
  std::atomic<int64_t> step_{0};
};

// ---------------------------------------------------------------------------------
// O4: decentralized, low precision, synchronous (compressed ring gossip)
// ---------------------------------------------------------------------------------
class DecentralizedLowPrecisionSynchronous : public CommOp {
 public:
  DecentralizedLowPrecisionSynchronous(std::shared_ptr<Communicator> c, PeerSelectionMode mode, std::string method,
                                       TensorPtr w, TensorPtr l, TensorPtr r)
      : comm_(std::move(c)), mode_(mode), method_(std::move(method)), w_(std::move(w)), l_(std::move(l)),
        r_(std::move(r)) {
    BAGUA_CHECK(mode_ == PeerSelectionMode::Ring, Bucket,
                "low precision decentralized op supports peer_selection_mode ring only");
    BAGUA_CHECK(method_ == "MinMaxUInt8", Bucket, "unsupported compression `" << method_ << "`");
  }

  void execute_background_communication(const BucketPtr& bucket) override {
    OpFrame f(bucket, *comm_, false, false);
    auto w = w_->raw(), l = l_->raw(), r = r_->raw();
    comm_->execute_communication(*f.ct.raw, true, true, true, [&](SingleCommunicator& c, RawTensor& t) {
      const uint64_t s = c.stream();
      if (PeerArena* a = fused_arena(c, t)) {
        const int64_t n = t.num_elements_allocated();
        if (w->num_elements_allocated() == n && l->num_elements_allocated() == n &&
            r->num_elements_allocated() == n &&
            fused::lp_ring(*a, t.data_ptr(), w->data_ptr(), l->data_ptr(), r->data_ptr(), n, t.dtype(),
                           (cudaStream_t)s)) {
          note_fused();
          return;
        }
        note_fallback();
      }
      tensor_ops::addmul_inplace(t, *l, 1.0f / 3.0f, s);
      tensor_ops::addmul_inplace(t, *r, 1.0f / 3.0f, s);
      tensor_ops::addmul_inplace(t, *w, -5.0f / 3.0f, s);
      auto compressed = tensor_ops::compress(t, method_, 1, s, -1);
      auto lrecv = PoolRawTensor::allocate(t.device_id(), DType::U8, compressed->num_elements_allocated(), s);
      auto rrecv = PoolRawTensor::allocate(t.device_id(), DType::U8, compressed->num_elements_allocated(), s);
      const int left = (c.rank() + c.nranks() - 1) % c.nranks();
      const int right = (c.rank() + 1) % c.nranks();
      {
        GroupGuard g(c);
        c.send(*compressed, left);
        c.send(*compressed, right);
        c.recv(*lrecv, left);
        c.recv(*rrecv, right);
      }
      tensor_ops::decompress_from(t, method_, 1, *lrecv, s);
      tensor_ops::add_inplace(*l, t, s);
      tensor_ops::decompress_from(t, method_, 1, *rrecv, s);
      tensor_ops::add_inplace(*r, t, s);
      tensor_ops::decompress_from(t, method_, 1, *compressed, s);
      tensor_ops::add_inplace(t, *w, s);
      tensor_ops::clone_from(*w, t, s);
    });
    f.finish();
  }
  std::string describe() const override {
    return "DecentralizedLowPrecisionSynchronous{peer_selection_mode=ring, compression=" + method_ + "}";
  }

 private:
  std::shared_ptr<Communicator> comm_;
  PeerSelectionMode mode_;
  std::string method_;
  TensorPtr w_, l_, r_;
};

// ---------------------------------------------------------------------------------
// O5: decentralized, full precision, asynchronous (async model averaging)
// ---------------------------------------------------------------------------------
class DecentralizedFullPrecisionAsynchronous : public CommOp {
 public:
  DecentralizedFullPrecisionAsynchronous(std::shared_ptr<Communicator> c, PeerSelectionMode mode,
                                         uint64_t torch_stream)
      : comm_(std::move(c)), mode_(mode), torch_stream_(torch_stream) {
    BAGUA_CHECK(mode_ == PeerSelectionMode::All, Bucket,
                "asynchronous decentralized op supports peer_selection_mode all only");
    BAGUA_CHECK(comm_->kind() == Communicator::Kind::Single, Communicator,
                "asynchronous op only accepts non-hierarchical communicator");
  }

  void execute_background_communication(const BucketPtr& bucket) override {
    const uint64_t t0 = now_us_steady();
    OpFrame f(bucket, *comm_, false, false);
    const uint64_t comm_stream = comm_->stream();
    RawTensor& t = *f.ct.raw;
    const bool gpu = t.device_id() >= 0;
    auto temp = PoolRawTensor::allocate(t.device_id(), t.dtype(), t.num_elements_allocated(), comm_stream);
    auto reduced = PoolRawTensor::allocate(t.device_id(), t.dtype(), t.num_elements_allocated(), comm_stream);
    SingleCommunicator& c = *comm_->internode();

    // Snapshot the weights on the training stream, then hand over to the comm stream.
    tensor_ops::clone_from(*temp, t, gpu ? torch_stream_ : 0);
    std::unique_ptr<EventLease> ev1, ev2, ev3;
    if (gpu) {
      ev1 = EventPool::instance().take();
      BAGUA_CUDA_CHECK(cudaEventRecord(ev1->get(), (cudaStream_t)torch_stream_));
      BAGUA_CUDA_CHECK(cudaStreamWaitEvent((cudaStream_t)comm_stream, ev1->get(), 0));
    }
    if (c.check_abort()) {
      f.finish();
      return;
    }
    bool done = false;
    if (PeerArena* a = fused_arena(c, t)) {
      if (fused::allreduce(*a, temp->data_ptr(), reduced->data_ptr(), t.num_elements_allocated(), t.dtype(), 1.0f,
                           (cudaStream_t)comm_stream)) {
        note_fused();
        done = true;
      } else {
        note_fallback();
      }
    }
    if (!done) c.allreduce(*temp, *reduced, ReductionOp::SUM);
    if (gpu) {
      ev2 = EventPool::instance().take();
      BAGUA_CUDA_CHECK(cudaEventRecord(ev2->get(), (cudaStream_t)comm_stream));
      BAGUA_CUDA_CHECK(cudaEventSynchronize(ev2->get()));
    }
    if (c.check_abort()) {
      f.finish();
      return;
    }
    if (gpu) {
      ev3 = EventPool::instance().take();
      BAGUA_CUDA_CHECK(cudaEventRecord(ev3->get(), (cudaStream_t)torch_stream_));
      BAGUA_CUDA_CHECK(cudaStreamWaitEvent((cudaStream_t)comm_stream, ev3->get(), 0));
    }
    tensor_ops::async_model_average(t, *reduced, *temp, (float)c.nranks(), comm_stream);
    if (gpu) BAGUA_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)comm_stream));
    f.finish();
    BAGUA_LOG(Debug, "async model average update cost: " << fmt_double((now_us_steady() - t0) / 1000.0) << " ms");
  }
  std::string describe() const override { return "DecentralizedFullPrecisionAsynchronous{peer_selection_mode=all}"; }

 private:
  std::shared_ptr<Communicator> comm_;
  PeerSelectionMode mode_;
  uint64_t torch_stream_;
};

// ---------------------------------------------------------------------------------
// O6: user callback
// ---------------------------------------------------------------------------------
class CallbackOp : public CommOp {
 public:
  CallbackOp(std::function<void(const std::string&)> call, std::string label)
      : call_(std::move(call)), label_(std::move(label)) {}
  void execute_background_communication(const BucketPtr& bucket) override {
    try {
      call_(bucket->name());
    } catch (const std::exception& e) {
      // like the reference (python_ffi_op.rs:18-23): errors are logged, not raised
      BAGUA_LOG(Error, "python op error: " << e.what());
    }
  }
  std::string describe() const override { return "PythonFFIOp{" + label_ + "}"; }

 private:
  std::function<void(const std::string&)> call_;
  std::string label_;
};

}  // namespace

std::shared_ptr<CommOp> make_centralized_full_precision_op(std::shared_ptr<Communicator> comm, bool average,
                                                           bool scattergather) {
  return std::make_shared<CentralizedFullPrecisionSynchronous>(std::move(comm), average, scattergather);
}
std::shared_ptr<CommOp> make_centralized_low_precision_op(std::shared_ptr<Communicator> comm, bool average,
                                                          const std::string& compression) {
  return std::make_shared<CentralizedLowPrecisionSynchronous>(std::move(comm), average, compression);
}
std::shared_ptr<CommOp> make_decentralized_full_precision_op(std::shared_ptr<Communicator> comm,
                                                             PeerSelectionMode mode, TensorPtr peer_weight) {
  return std::make_shared<DecentralizedFullPrecisionSynchronous>(std::move(comm), mode, std::move(peer_weight));
}
std::shared_ptr<CommOp> make_decentralized_low_precision_op(std::shared_ptr<Communicator> comm,
                                                            PeerSelectionMode mode, const std::string& compression,
                                                            TensorPtr weight, TensorPtr left, TensorPtr right) {
  return std::make_shared<DecentralizedLowPrecisionSynchronous>(std::move(comm), mode, compression, std::move(weight),
                                                                std::move(left), std::move(right));
}
std::shared_ptr<CommOp> make_decentralized_async_op(std::shared_ptr<Communicator> comm, PeerSelectionMode mode,
                                                    uint64_t torch_stream) {
  return std::make_shared<DecentralizedFullPrecisionAsynchronous>(std::move(comm), mode, torch_stream);
}
std::shared_ptr<CommOp> make_callback_op(std::function<void(const std::string&)> call, std::string label) {
  return std::make_shared<CallbackOp>(std::move(call), std::move(label));
}

}  // namespace bagua
