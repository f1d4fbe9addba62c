#include "communicator.h"

#include <cuda_runtime.h>

#include "../kernels/fused.h"
#include "../runtime/stats.h"
#include "arena.h"

namespace bagua {

namespace {
// Live communicators, for check_all_device_status().
std::mutex g_comms_mu;
std::vector<SingleCommunicator*> g_comms;

void same_kind(const RawTensor& a, const RawTensor& b, const char* what) {
  BAGUA_CHECK(a.dtype() == b.dtype(), Communicator, what << ": send and recv dtypes differ");
  BAGUA_CHECK(a.device_id() == b.device_id(), Communicator, what << ": send and recv devices differ");
}
}  // namespace

SingleCommunicator::SingleCommunicator(int rank, int nranks, int device_id, uint64_t stream,
                                       const std::string& unique_id)
    : rank_(rank), nranks_(nranks), device_id_(device_id), stream_(stream) {
  BAGUA_CHECK(nranks >= 1 && rank >= 0 && rank < nranks, Communicator, "invalid rank " << rank << " / " << nranks);
  if (is_solo_unique_id(unique_id)) {
    BAGUA_CHECK(nranks == 1, Communicator, "the one-rank transport needs nranks = 1");
    transport_ = make_solo_transport(device_id, stream);
  } else if (is_c10d_unique_id(unique_id)) {
    BAGUA_CHECK(device_id < 0, Communicator, "the c10d transport works on host memory: pass device_id = -1");
    transport_ = make_c10d_transport(rank, nranks, unique_id.substr(5));
  } else {
    BAGUA_CHECK(device_id >= 0, Communicator, "an NCCL communicator needs a CUDA device id");
    transport_ = make_nccl_transport(rank, nranks, device_id, stream, unique_id);
  }
  fused_enabled_ = env_long("BAGUA_B200_FUSED", 1) != 0;
  p2p_collectives_ = env_long("BAGUA_B200_P2P_COLLECTIVES", 0) != 0;
  std::lock_guard<std::mutex> g(g_comms_mu);
  g_comms.push_back(this);
}

SingleCommunicator::~SingleCommunicator() {
  {
    std::lock_guard<std::mutex> g(g_comms_mu);
    for (size_t i = 0; i < g_comms.size(); ++i)
      if (g_comms[i] == this) {
        g_comms.erase(g_comms.begin() + (long)i);
        break;
      }
  }
  arena_.reset();
  transport_.reset();
}

void SingleCommunicator::abort() {
  aborted_.store(true, std::memory_order_release);
  {
    // fused kernels of this rank that wait for a peer see the word at their next poll and return
    // (reference: abort() also stops the in-flight NCCL kernels, communicators/mod.rs:456-471)
    std::lock_guard<std::mutex> g(arena_mu_);
    if (arena_) arena_->poison();
  }
  transport_->abort();
}

void SingleCommunicator::check_all_device_status() {
  std::lock_guard<std::mutex> g(g_comms_mu);
  for (SingleCommunicator* c : g_comms) c->check_device_status(/*try_only=*/true);
}

void SingleCommunicator::check_live() const {
  if (check_abort()) throw BaguaError(ErrorKind::Communicator, "communicator was aborted");
}

void SingleCommunicator::check_rank(int r, const char* what) const {
  BAGUA_CHECK(r >= 0 && r < nranks_, Communicator, what << " rank " << r << " out of range (" << nranks_ << " ranks)");
}

PeerArena* SingleCommunicator::arena() {
  if (device_id_ < 0 || nranks_ < 2 || nranks_ > kArenaMaxRanks || !fused_enabled_) return nullptr;
  std::lock_guard<std::mutex> g(arena_mu_);
  if (!arena_tried_) {
    arena_tried_ = true;
    try {
      arena_ = std::make_unique<PeerArena>(*transport_, rank_, nranks_, device_id_, (cudaStream_t)stream_);
    } catch (const std::exception& e) {
      // Mapping peers failed (no P2P between the devices, IPC disabled ...).  Every
      // rank sees the same topology, so every rank lands here and the library path
      // is used consistently.
      BAGUA_LOG(Warn, "peer arena unavailable, using library collectives: " << e.what());
      arena_.reset();
    }
  }
  return arena_.get();
}

PeerArena* SingleCommunicator::p2p_arena() {
  if (!p2p_collectives_ || group_depth_ > 0) return nullptr;
  return arena();
}

namespace {
// Scale of a reduction the peer-memory kernels implement; 0 when they do not.
float p2p_scale(ReductionOp op, int nranks) {
  if (op == ReductionOp::SUM) return 1.0f;
  if (op == ReductionOp::AVG) return 1.0f / (float)nranks;
  return 0.0f;
}
}  // namespace

void SingleCommunicator::check_device_status(bool try_only) {
  // try_only: a communicator whose arena is being set up right now (a collective that may take a
  // while) is skipped instead of waited for; its record is looked at by the next check
  std::unique_lock<std::mutex> g(arena_mu_, std::defer_lock);
  if (try_only) {
    if (!g.try_lock()) return;
  } else {
    g.lock();
  }
  if (!arena_) return;
  DeviceStatus s = arena_->read_status();
  if (s.code == 0) return;
  aborted_.store(true, std::memory_order_release);
  arena_->clear_status();  // reported once; from here on the communicator answers "aborted"
  std::ostringstream o;
  if (s.code == 4) {
    o << "alltoall_v: rank " << s.peer << " announced a segment of " << s.seen << " bytes for rank " << rank_
      << ", which expected another size (op " << s.epoch << "); the communicator is now aborted";
    throw BaguaError(ErrorKind::Communicator, o.str());
  }
  static const char* what[] = {"", "wait for a peer to finish its previous op", "wait for a peer's data signal",
                               "grid barrier"};
  o << "a device-side " << (s.code < 4 ? what[s.code] : "wait") << " ran out after " << fmt_double(arena_->deadline_ms())
    << " ms (rank " << rank_ << ", peer " << s.peer << ", phase " << s.phase << ", block " << s.block << ", epoch "
    << s.epoch << ", last value seen " << s.seen << "); the communicator is now aborted";
  throw BaguaError(ErrorKind::Communicator, o.str());
}

// ---- collectives ------------------------------------------------------------------
void SingleCommunicator::allreduce(const RawTensor& send, RawTensor& recv, ReductionOp op) {
  check_live();
  same_kind(send, recv, "allreduce");
  BAGUA_CHECK(send.num_elements_allocated() == recv.num_elements_allocated(), Communicator,
              "allreduce: send and recv sizes differ");
  if (PeerArena* a = p2p_arena()) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::allreduce(*a, send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(),
                                          send.dtype(), scale, (cudaStream_t)stream_))
      return;
  }
  transport_->allreduce(send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(), send.dtype(), op);
}
void SingleCommunicator::allreduce_inplace(RawTensor& t, ReductionOp op, bool engine_op) {
  check_live();
  PeerArena* a = nullptr;
  if (engine_op && t.device_id() >= 0 && group_depth_ == 0) {
    a = arena();
    if (a) {
      check_device_status();
      check_live();
    }
  } else {
    a = p2p_arena();
  }
  if (a) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::allreduce(*a, t.data_ptr(), t.data_ptr(), t.num_elements_allocated(), t.dtype(), scale,
                                          (cudaStream_t)stream_, engine_op)) {
      if (engine_op) EngineStats::global().fused_launches++;
      return;
    }
    if (engine_op) EngineStats::global().library_fallbacks++;
  }
  transport_->allreduce(t.data_ptr(), t.data_ptr(), t.num_elements_allocated(), t.dtype(), op);
}
void SingleCommunicator::broadcast(RawTensor& t, int root) {
  check_live();
  check_rank(root, "broadcast: root");
  if (PeerArena* a = p2p_arena())
    if (fused::broadcast(*a, t.data_ptr(), t.bytes_allocated(), root, (cudaStream_t)stream_)) return;
  transport_->broadcast(t.data_ptr(), t.num_elements_allocated(), t.dtype(), root);
}
void SingleCommunicator::reduce(const RawTensor& send, RawTensor& recv, int dst, ReductionOp op) {
  check_live();
  same_kind(send, recv, "reduce");
  check_rank(dst, "reduce: destination");
  BAGUA_CHECK(send.num_elements_allocated() == recv.num_elements_allocated(), Communicator,
              "reduce: send and recv sizes differ");
  if (PeerArena* a = p2p_arena()) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::reduce(*a, send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(),
                                       send.dtype(), scale, dst, (cudaStream_t)stream_))
      return;
  }
  transport_->reduce(send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(), send.dtype(), dst, op);
}
void SingleCommunicator::reduce_inplace(RawTensor& t, int dst, ReductionOp op) {
  check_live();
  check_rank(dst, "reduce: destination");
  if (PeerArena* a = p2p_arena()) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::reduce(*a, t.data_ptr(), t.data_ptr(), t.num_elements_allocated(), t.dtype(), scale,
                                       dst, (cudaStream_t)stream_))
      return;
  }
  transport_->reduce(t.data_ptr(), t.data_ptr(), t.num_elements_allocated(), t.dtype(), dst, op);
}
void SingleCommunicator::send(const RawTensor& t, int peer) {
  check_live();
  check_rank(peer, "send: peer");
  transport_->send(t.data_ptr(), t.num_elements_allocated(), t.dtype(), peer);
}
void SingleCommunicator::recv(RawTensor& t, int peer) {
  check_live();
  check_rank(peer, "recv: peer");
  transport_->recv(t.data_ptr(), t.num_elements_allocated(), t.dtype(), peer);
}
void SingleCommunicator::alltoall(const RawTensor& send, RawTensor& recv) {
  check_live();
  same_kind(send, recv, "alltoall");
  BAGUA_CHECK(send.num_elements_allocated() == recv.num_elements_allocated(), Communicator,
              "alltoall: send and recv sizes differ");
  BAGUA_CHECK(send.num_elements_allocated() % nranks_ == 0, Communicator,
              "alltoall: tensor size must be divisible by the number of ranks");
  if (PeerArena* a = p2p_arena())
    if (fused::alltoall(*a, send.data_ptr(), recv.data_ptr(), send.bytes_allocated() / (size_t)nranks_,
                        (cudaStream_t)stream_))
      return;
  transport_->alltoall(send.data_ptr(), recv.data_ptr(), send.num_elements_allocated() / nranks_, send.dtype());
}
void SingleCommunicator::alltoall_inplace(RawTensor& t) {
  check_live();
  BAGUA_CHECK(t.num_elements_allocated() % nranks_ == 0, Communicator,
              "alltoall: tensor size must be divisible by the number of ranks");
  if (PeerArena* a = p2p_arena())
    if (fused::alltoall(*a, t.data_ptr(), t.data_ptr(), t.bytes_allocated() / (size_t)nranks_, (cudaStream_t)stream_))
      return;
  // Exchange out of a copy: slot p is both what goes to p and where p's data lands.
  auto tmp = PoolRawTensor::allocate(t.device_id(), t.dtype(), t.num_elements_allocated(), stream_);
  kernels::copy_bytes(tmp->data_ptr(), t.data_ptr(), t.bytes_allocated(), t.ctx(stream_));
  transport_->alltoall(tmp->data_ptr(), t.data_ptr(), t.num_elements_allocated() / nranks_, t.dtype());
}
void SingleCommunicator::alltoall_v(const RawTensor& send, const std::vector<int64_t>& sc,
                                    const std::vector<int64_t>& sd, RawTensor& recv, const std::vector<int64_t>& rc,
                                    const std::vector<int64_t>& rd) {
  check_live();
  same_kind(send, recv, "alltoall_v");
  BAGUA_CHECK((int)sc.size() == nranks_ && (int)sd.size() == nranks_ && (int)rc.size() == nranks_ &&
                  (int)rd.size() == nranks_,
              Communicator, "alltoall_v: counts and displacements must have one entry per rank");
  for (int p = 0; p < nranks_; ++p) {
    BAGUA_CHECK(sc[p] >= 0 && sd[p] >= 0 && sd[p] + sc[p] <= send.num_elements_allocated(), Communicator,
                "alltoall_v: send range of rank " << p << " is outside the tensor");
    BAGUA_CHECK(rc[p] >= 0 && rd[p] >= 0 && rd[p] + rc[p] <= recv.num_elements_allocated(), Communicator,
                "alltoall_v: recv range of rank " << p << " is outside the tensor");
  }
  if (PeerArena* a = p2p_arena())
    if (fused::alltoall_v(*a, send.data_ptr(), send.bytes_allocated(), sc.data(), sd.data(), recv.data_ptr(),
                          recv.bytes_allocated(), rc.data(), rd.data(), dtype_bytes(send.dtype()), (cudaStream_t)stream_))
      return;
  transport_->alltoall_v(send.data_ptr(), sc, sd, recv.data_ptr(), rc, rd, send.dtype());
}
void SingleCommunicator::allgather(const RawTensor& send, RawTensor& recv) {
  check_live();
  same_kind(send, recv, "allgather");
  BAGUA_CHECK(send.num_elements_allocated() * nranks_ == recv.num_elements_allocated(), Communicator,
              "allgather: recv must hold nranks * send elements");
  if (PeerArena* a = p2p_arena())
    if (fused::allgather(*a, send.data_ptr(), recv.data_ptr(), send.bytes_allocated(), (cudaStream_t)stream_)) return;
  transport_->allgather(send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(), send.dtype());
}
void SingleCommunicator::allgather_inplace(RawTensor& t) {
  check_live();
  BAGUA_CHECK(t.num_elements_allocated() % nranks_ == 0, Communicator,
              "allgather: tensor size must be divisible by the number of ranks");
  const int64_t count = t.num_elements_allocated() / nranks_;
  const size_t es = dtype_bytes(t.dtype());
  if (PeerArena* a = p2p_arena())
    if (fused::allgather(*a, (char*)t.data_ptr() + (size_t)rank_ * count * es, t.data_ptr(), (size_t)count * es,
                         (cudaStream_t)stream_))
      return;
  transport_->allgather((char*)t.data_ptr() + (size_t)rank_ * count * es, t.data_ptr(), count, t.dtype());
}
void SingleCommunicator::gather(const RawTensor& send, RawTensor& recv, int dst) {
  check_live();
  same_kind(send, recv, "gather");
  check_rank(dst, "gather: destination");
  if (rank_ == dst)
    BAGUA_CHECK(send.num_elements_allocated() * nranks_ == recv.num_elements_allocated(), Communicator,
                "gather: recv on the root must hold nranks * send elements");
  if (PeerArena* a = p2p_arena())
    if (fused::gather(*a, send.data_ptr(), recv.data_ptr(), send.bytes_allocated(), dst, (cudaStream_t)stream_)) return;
  transport_->gather(send.data_ptr(), recv.data_ptr(), send.num_elements_allocated(), send.dtype(), dst);
}
void SingleCommunicator::gather_inplace(RawTensor& t, int64_t count, int dst) {
  check_live();
  check_rank(dst, "gather: destination");
  BAGUA_CHECK(count >= 0, Communicator, "gather_inplace: negative count");
  if (rank_ == dst)
    BAGUA_CHECK(t.num_elements_allocated() == count * nranks_, Communicator,
                "gather_inplace: the root tensor must hold count * nranks elements");
  else
    BAGUA_CHECK(t.num_elements_allocated() >= count, Communicator, "gather_inplace: tensor smaller than count");
  const size_t es = dtype_bytes(t.dtype());
  const void* src = rank_ == dst ? (char*)t.data_ptr() + (size_t)rank_ * count * es : t.data_ptr();
  if (PeerArena* a = p2p_arena())
    if (fused::gather(*a, src, t.data_ptr(), (size_t)count * es, dst, (cudaStream_t)stream_)) return;
  transport_->gather(src, t.data_ptr(), count, t.dtype(), dst);
}
void SingleCommunicator::scatter(const RawTensor& send, RawTensor& recv, int src) {
  check_live();
  same_kind(send, recv, "scatter");
  check_rank(src, "scatter: source");
  if (rank_ == src)
    BAGUA_CHECK(recv.num_elements_allocated() * nranks_ == send.num_elements_allocated(), Communicator,
                "scatter: send on the root must hold nranks * recv elements");
  if (PeerArena* a = p2p_arena())
    if (fused::scatter(*a, send.data_ptr(), recv.data_ptr(), recv.bytes_allocated(), src, (cudaStream_t)stream_)) return;
  transport_->scatter(send.data_ptr(), recv.data_ptr(), recv.num_elements_allocated(), recv.dtype(), src);
}
void SingleCommunicator::scatter_inplace(RawTensor& t, int64_t count, int src) {
  check_live();
  check_rank(src, "scatter: source");
  BAGUA_CHECK(count >= 0, Communicator, "scatter_inplace: negative count");
  if (rank_ == src)
    BAGUA_CHECK(t.num_elements_allocated() == count * nranks_, Communicator,
                "scatter_inplace: the root tensor must hold count * nranks elements");
  else
    BAGUA_CHECK(t.num_elements_allocated() >= count, Communicator, "scatter_inplace: tensor smaller than count");
  const size_t es = dtype_bytes(t.dtype());
  void* dst = rank_ == src ? (char*)t.data_ptr() + (size_t)rank_ * count * es : t.data_ptr();
  if (PeerArena* a = p2p_arena())
    if (fused::scatter(*a, t.data_ptr(), dst, (size_t)count * es, src, (cudaStream_t)stream_)) return;
  transport_->scatter(t.data_ptr(), dst, count, t.dtype(), src);
}
void SingleCommunicator::reduce_scatter(const RawTensor& send, RawTensor& recv, ReductionOp op) {
  check_live();
  same_kind(send, recv, "reduce_scatter");
  BAGUA_CHECK(recv.num_elements_allocated() * nranks_ == send.num_elements_allocated(), Communicator,
              "reduce_scatter: send must hold nranks * recv elements");
  if (PeerArena* a = p2p_arena()) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::reduce_scatter(*a, send.data_ptr(), recv.data_ptr(), recv.num_elements_allocated(),
                                               send.dtype(), scale, (cudaStream_t)stream_))
      return;
  }
  transport_->reduce_scatter(send.data_ptr(), recv.data_ptr(), recv.num_elements_allocated(), send.dtype(), op);
}
void SingleCommunicator::reduce_scatter_inplace(RawTensor& t, ReductionOp op) {
  check_live();
  BAGUA_CHECK(t.num_elements_allocated() % nranks_ == 0, Communicator,
              "reduce_scatter: tensor size must be divisible by the number of ranks");
  const int64_t count = t.num_elements_allocated() / nranks_;
  const size_t es = dtype_bytes(t.dtype());
  if (PeerArena* a = p2p_arena()) {
    const float scale = p2p_scale(op, nranks_);
    if (scale != 0.0f && fused::reduce_scatter(*a, t.data_ptr(), (char*)t.data_ptr() + (size_t)rank_ * count * es, count,
                                               t.dtype(), scale, (cudaStream_t)stream_))
      return;
  }
  transport_->reduce_scatter(t.data_ptr(), (char*)t.data_ptr() + (size_t)rank_ * count * es, count, t.dtype(), op);
}
void SingleCommunicator::barrier() {
  check_live();
  if (PeerArena* a = p2p_arena())
    if (fused::barrier(*a, (cudaStream_t)stream_)) {
      // like the library barrier, return only once every rank has arrived
      BAGUA_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
      check_device_status();
      return;
    }
  transport_->barrier();
}

int64_t SingleCommunicator::agree_inter_nranks(int64_t mine) {
  if (inter_nranks_ >= 0) return inter_nranks_;
  check_live();
  int64_t v = rank_ == 0 ? mine : 0;
  if (nranks_ > 1) {
    auto buf = PoolRawTensor::allocate(device_id_, DType::I64, 1, stream_);
    if (device_id_ >= 0) {
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(buf->data_ptr(), &v, sizeof(v), cudaMemcpyHostToDevice, (cudaStream_t)stream_));
      transport_->broadcast(buf->data_ptr(), 1, DType::I64, 0);
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(&v, buf->data_ptr(), sizeof(v), cudaMemcpyDeviceToHost, (cudaStream_t)stream_));
      BAGUA_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
    } else {
      std::memcpy(buf->data_ptr(), &v, sizeof(v));
      transport_->broadcast(buf->data_ptr(), 1, DType::I64, 0);
      std::memcpy(&v, buf->data_ptr(), sizeof(v));
    }
  }
  inter_nranks_ = v;
  return v;
}

// ---- two-level ----------------------------------------------------------------------
std::shared_ptr<Communicator> Communicator::create(SingleCommPtr internode, SingleCommPtr intranode,
                                                   bool hierarchical) {
  auto c = std::make_shared<Communicator>();
  if (!hierarchical) {
    BAGUA_CHECK(internode != nullptr, Communicator, "inter node communicator must be given in non-hierarchical mode");
    c->kind_ = Kind::Single;
    c->internode_ = std::move(internode);
    return c;
  }
  BAGUA_CHECK(intranode != nullptr, Communicator, "intra node communicator must be given in hierarchical mode");
  if (intranode->rank() == 0)
    BAGUA_CHECK(internode != nullptr, Communicator,
                "inter node communicator must be given on the leader GPU in hierarchical mode");
  // Collective over the node on first use: is the node the whole job?
  static const bool flat_ok = env_long("BAGUA_B200_HIERARCHICAL_FLAT", 1) != 0;
  if (flat_ok && intranode->agree_inter_nranks(internode ? internode->nranks() : 0) == 1)
    c->solo_ = std::make_shared<SingleCommunicator>(0, 1, intranode->device_id(), intranode->stream(), "solo");
  if (intranode->rank() == 0) {
    BAGUA_CHECK(intranode->stream() == internode->stream(), Communicator,
                "intra node communicator should use the same stream as the inter node communicator");
    BAGUA_CHECK(intranode->device_id() == internode->device_id(), Communicator,
                "intra node and inter node communicators must be on the same device");
    c->kind_ = Kind::HierarchicalLeader;
    c->internode_ = std::move(internode);
    c->intranode_ = std::move(intranode);
  } else {
    c->kind_ = Kind::HierarchicalWorker;
    c->intranode_ = std::move(intranode);
  }
  return c;
}

uint64_t Communicator::stream() const {
  return kind_ == Kind::HierarchicalWorker ? intranode_->stream() : internode_->stream();
}

void Communicator::execute_communication(RawTensor& t, bool intranode_average, bool pre, bool post,
                                         const std::function<void(SingleCommunicator&, RawTensor&)>& hook) {
  if (solo_ && kind_ != Kind::Single && pre && post) {
    // one node is the whole job: reduce to the leader + broadcast from it = one all-reduce (the
    // fused kernel when this communicator's collectives run over peer memory), and the
    // inter-node step over one rank is local, deterministic work that every rank does itself
    intranode_->allreduce_inplace(t, intranode_average ? ReductionOp::AVG : ReductionOp::SUM, /*engine_op=*/true);
    hook(*solo_, t);
    return;
  }
  switch (kind_) {
    case Kind::Single: hook(*internode_, t); return;
    case Kind::HierarchicalLeader:
      if (pre) intranode_->reduce_inplace(t, 0, intranode_average ? ReductionOp::AVG : ReductionOp::SUM);
      hook(*internode_, t);
      if (post) intranode_->broadcast(t, 0);
      return;
    case Kind::HierarchicalWorker:
      if (pre) intranode_->reduce_inplace(t, 0, intranode_average ? ReductionOp::AVG : ReductionOp::SUM);
      if (post) intranode_->broadcast(t, 0);
      return;
  }
}

}  // namespace bagua
