// c10d (gloo) transport over host memory.
//
// The process group is looked up by name in torch's group registry, so the Python layer
// only passes "c10d:<group_name>" where the GPU path passes an NCCL unique id.  Raw
// pointers are wrapped with `at::from_blob` (no copies).  AVG is SUM followed by a
// division, since gloo has no averaging reduction.
#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>

#include <functional>

#include "transport.h"

namespace bagua {

namespace {

at::ScalarType to_at(DType dt) {
  switch (dt) {
    case DType::F32: return at::kFloat;
    case DType::F16: return at::kHalf;
    case DType::U8: return at::kByte;
    case DType::I64: return at::kLong;
    case DType::BF16: return at::kBFloat16;
    case DType::U64: return at::kLong;  // bit pattern only; no arithmetic collectives on U64
  }
  throw BaguaError(ErrorKind::Communicator, "unsupport tensor data type.");
}

c10d::ReduceOp to_c10d(ReductionOp op) {
  switch (op) {
    case ReductionOp::SUM: return c10d::ReduceOp::SUM;
    case ReductionOp::AVG: return c10d::ReduceOp::SUM;  // divided afterwards
    case ReductionOp::PROD: return c10d::ReduceOp::PRODUCT;
    case ReductionOp::MIN: return c10d::ReduceOp::MIN;
    case ReductionOp::MAX: return c10d::ReduceOp::MAX;
    case ReductionOp::BOR: return c10d::ReduceOp::BOR;
    case ReductionOp::BAND: return c10d::ReduceOp::BAND;
    case ReductionOp::BXOR: return c10d::ReduceOp::BXOR;
    default:
      throw BaguaError(ErrorKind::Communicator,
                       "reduction op " + std::to_string((int)op) + " is not available on the c10d transport");
  }
}

at::Tensor wrap(const void* p, int64_t count, DType dt) {
  return at::from_blob(const_cast<void*>(p), {count}, at::TensorOptions().dtype(to_at(dt)).device(at::kCPU));
}

void apply_avg(at::Tensor t, int nranks) {
  if (at::isFloatingType(t.scalar_type()))
    t.div_(nranks);
  else
    t.floor_divide_(nranks);
}

class C10dTransport : public Transport {
 public:
  C10dTransport(int rank, int nranks, const std::string& group)
      : rank_(rank), nranks_(nranks), pg_(c10d::resolve_process_group(group)) {
    BAGUA_CHECK(pg_->getRank() == rank && pg_->getSize() == nranks, Communicator,
                "process group `" << group << "` has rank/size " << pg_->getRank() << "/" << pg_->getSize()
                                  << ", communicator was given " << rank << "/" << nranks);
  }
  int rank() const override { return rank_; }
  int nranks() const override { return nranks_; }
  const char* kind() const override { return "c10d"; }

  void allreduce(const void* send, void* recv, int64_t count, DType dt, ReductionOp op) override {
    check_abort();
    if (send != recv) std::memcpy(recv, send, (size_t)count * dtype_bytes(dt));
    std::vector<at::Tensor> ts{wrap(recv, count, dt)};
    c10d::AllreduceOptions o;
    o.reduceOp = to_c10d(op);
    pg_->allreduce(ts, o)->wait();
    if (op == ReductionOp::AVG) apply_avg(ts[0], nranks_);
  }
  void broadcast(void* buf, int64_t count, DType dt, int root) override {
    check_abort();
    std::vector<at::Tensor> ts{wrap(buf, count, dt)};
    c10d::BroadcastOptions o;
    o.rootRank = root;
    pg_->broadcast(ts, o)->wait();
  }
  void reduce(const void* send, void* recv, int64_t count, DType dt, int root, ReductionOp op) override {
    check_abort();
    // gloo reduces in place; non-root ranks must not have their recv buffer touched.
    at::Tensor work = (rank_ == root) ? wrap(recv, count, dt) : wrap(send, count, dt).clone();
    if (rank_ == root && send != recv) std::memcpy(recv, send, (size_t)count * dtype_bytes(dt));
    std::vector<at::Tensor> ts{work};
    c10d::ReduceOptions o;
    o.reduceOp = to_c10d(op);
    o.rootRank = root;
    pg_->reduce(ts, o)->wait();
    if (op == ReductionOp::AVG && rank_ == root) apply_avg(work, nranks_);
  }
  void send(const void* buf, int64_t count, DType dt, int peer) override {
    check_abort();
    auto fn = [this, buf, count, dt, peer]() {
      std::vector<at::Tensor> ts{wrap(buf, count, dt)};
      return pg_->send(ts, peer, 0);
    };
    if (group_depth_ > 0)
      pending_sends_.push_back(fn);
    else
      fn()->wait();
  }
  void recv(void* buf, int64_t count, DType dt, int peer) override {
    check_abort();
    auto fn = [this, buf, count, dt, peer]() {
      std::vector<at::Tensor> ts{wrap(buf, count, dt)};
      return pg_->recv(ts, peer, 0);
    };
    if (group_depth_ > 0)
      pending_recvs_.push_back(fn);
    else
      fn()->wait();
  }
  void alltoall(const void* send, void* recv, int64_t count, DType dt) override {
    check_abort();
    at::Tensor in = wrap(send, count * nranks_, dt), out = wrap(recv, count * nranks_, dt);
    std::vector<int64_t> none;
    pg_->alltoall_base(out, in, none, none)->wait();
  }
  void alltoall_v(const void* send, const std::vector<int64_t>& sc, const std::vector<int64_t>& sd, void* recv,
                  const std::vector<int64_t>& rc, const std::vector<int64_t>& rd, DType dt) override {
    check_abort();
    // Pairwise exchange with explicit displacements (alltoall_base assumes packed layouts).
    const size_t es = dtype_bytes(dt);
    std::vector<c10::intrusive_ptr<c10d::Work>> works;
    for (int p = 0; p < nranks_; ++p) {
      if (p == rank_) continue;
      if (sc[p] > 0) {
        std::vector<at::Tensor> ts{wrap((const char*)send + (size_t)sd[p] * es, sc[p], dt)};
        works.push_back(pg_->send(ts, p, 1));
      }
    }
    for (int p = 0; p < nranks_; ++p) {
      if (p == rank_) continue;
      if (rc[p] > 0) {
        std::vector<at::Tensor> ts{wrap((char*)recv + (size_t)rd[p] * es, rc[p], dt)};
        works.push_back(pg_->recv(ts, p, 1));
      }
    }
    if (sc[rank_] > 0)
      std::memmove((char*)recv + (size_t)rd[rank_] * es, (const char*)send + (size_t)sd[rank_] * es,
                   (size_t)std::min(sc[rank_], rc[rank_]) * es);
    for (auto& w : works) w->wait();
  }
  void allgather(const void* send, void* recv, int64_t count, DType dt) override {
    check_abort();
    at::Tensor in = wrap(send, count, dt).clone();  // `send` may alias its slot in `recv`
    at::Tensor out = wrap(recv, count * nranks_, dt);
    pg_->_allgather_base(out, in)->wait();
  }
  void gather(const void* send, void* recv, int64_t count, DType dt, int root) override {
    check_abort();
    std::vector<at::Tensor> in{wrap(send, count, dt).clone()};
    std::vector<std::vector<at::Tensor>> out;
    if (rank_ == root) {
      out.emplace_back();
      for (int p = 0; p < nranks_; ++p)
        out[0].push_back(wrap((char*)recv + (size_t)p * count * dtype_bytes(dt), count, dt));
    }
    c10d::GatherOptions o;
    o.rootRank = root;
    pg_->gather(out, in, o)->wait();
  }
  void scatter(const void* send, void* recv, int64_t count, DType dt, int root) override {
    check_abort();
    std::vector<at::Tensor> out{wrap(recv, count, dt)};
    std::vector<std::vector<at::Tensor>> in;
    if (rank_ == root) {
      in.emplace_back();
      for (int p = 0; p < nranks_; ++p)
        in[0].push_back(wrap((const char*)send + (size_t)p * count * dtype_bytes(dt), count, dt).clone());
    }
    c10d::ScatterOptions o;
    o.rootRank = root;
    pg_->scatter(out, in, o)->wait();
  }
  void reduce_scatter(const void* send, void* recv, int64_t recv_count, DType dt, ReductionOp op) override {
    check_abort();
    // gloo has no reduce-scatter: all-reduce a copy and keep this rank's slice.
    at::Tensor work = wrap(send, recv_count * nranks_, dt).clone();
    std::vector<at::Tensor> ts{work};
    c10d::AllreduceOptions o;
    o.reduceOp = to_c10d(op);
    pg_->allreduce(ts, o)->wait();
    at::Tensor mine = work.narrow(0, (int64_t)rank_ * recv_count, recv_count);
    if (op == ReductionOp::AVG) apply_avg(mine, nranks_);
    std::memcpy(recv, mine.data_ptr(), (size_t)recv_count * dtype_bytes(dt));
  }
  void barrier() override {
    check_abort();
    pg_->barrier()->wait();
  }
  void group_start() override { ++group_depth_; }
  void group_end() override {
    if (--group_depth_ > 0) return;
    std::vector<c10::intrusive_ptr<c10d::Work>> works;
    for (auto& f : pending_sends_) works.push_back(f());
    for (auto& f : pending_recvs_) works.push_back(f());
    pending_sends_.clear();
    pending_recvs_.clear();
    for (auto& w : works) w->wait();
  }
  void abort() override { aborted_ = true; }

 private:
  void check_abort() const {
    if (aborted_) throw BaguaError(ErrorKind::Communicator, "communicator was aborted");
  }
  int rank_, nranks_;
  c10::intrusive_ptr<c10d::ProcessGroup> pg_;
  int group_depth_ = 0;
  std::vector<std::function<c10::intrusive_ptr<c10d::Work>()>> pending_sends_, pending_recvs_;
  std::atomic<bool> aborted_{false};
};

}  // namespace

std::unique_ptr<Transport> make_c10d_transport(int rank, int nranks, const std::string& group_name) {
  try {
    return std::make_unique<C10dTransport>(rank, nranks, group_name);
  } catch (const c10::Error& e) {
    throw BaguaError(ErrorKind::Communicator, std::string("cannot resolve process group: ") + e.what_without_backtrace());
  }
}

}  // namespace bagua
