// NCCL transport: every collective of the communicator API on one CUDA stream.
//
// Reference behaviour (bagua-core-internal/src/communicators/mod.rs): one NCCL
// communicator bound to a caller-supplied stream (10-17,44), bootstrap from a base64
// unique id (38-43,226-240), AVG as a native reduction, all-to-all as grouped
// send/recv, abort() on the communicator (456-467).
#include <cuda_runtime.h>
#include <nccl.h>

#include "base64.h"
#include "transport.h"

namespace bagua {

namespace {

ncclDataType_t to_nccl(DType dt) {
  switch (dt) {
    case DType::F32: return ncclFloat32;
    case DType::F16: return ncclFloat16;
    case DType::U8: return ncclUint8;
    case DType::I64: return ncclInt64;
    case DType::U64: return ncclUint64;
    case DType::BF16: return ncclBfloat16;
  }
  throw BaguaError(ErrorKind::Communicator, "unsupport tensor data type.");
}

ncclRedOp_t to_nccl(ReductionOp op) {
  switch (op) {
    case ReductionOp::SUM: return ncclSum;
    case ReductionOp::PROD: return ncclProd;
    case ReductionOp::MIN: return ncclMin;
    case ReductionOp::MAX: return ncclMax;
    case ReductionOp::AVG: return ncclAvg;
    default:
      throw BaguaError(ErrorKind::Communicator,
                       "reduction op " + std::to_string((int)op) + " is not available on the NCCL transport");
  }
}

class NcclTransport : public Transport {
 public:
  NcclTransport(int rank, int nranks, int device, uint64_t stream, const std::string& uid_b64)
      : rank_(rank), nranks_(nranks), device_(device), stream_((cudaStream_t)stream) {
    std::string raw = base64_decode(uid_b64);
    BAGUA_CHECK(raw.size() == sizeof(ncclUniqueId), Communicator,
                "nccl unique id must decode to " << sizeof(ncclUniqueId) << " bytes, got " << raw.size());
    ncclUniqueId id;
    std::memcpy(&id, raw.data(), sizeof(id));
    BAGUA_CUDA_CHECK(cudaSetDevice(device));
    BAGUA_NCCL_CHECK(ncclCommInitRank(&comm_, nranks, id, rank));
  }
  ~NcclTransport() override {
    if (comm_) {
      // Abort rather than destroy: destroy waits for outstanding work of every rank and
      // can block interpreter shutdown when a peer already left.
      ncclCommAbort(comm_);
      comm_ = nullptr;
    }
  }
  int rank() const override { return rank_; }
  int nranks() const override { return nranks_; }
  const char* kind() const override { return "nccl"; }

  void allreduce(const void* send, void* recv, int64_t count, DType dt, ReductionOp op) override {
    BAGUA_NCCL_CHECK(ncclAllReduce(send, recv, (size_t)count, to_nccl(dt), to_nccl(op), comm_, stream_));
  }
  void broadcast(void* buf, int64_t count, DType dt, int root) override {
    BAGUA_NCCL_CHECK(ncclBroadcast(buf, buf, (size_t)count, to_nccl(dt), root, comm_, stream_));
  }
  void reduce(const void* send, void* recv, int64_t count, DType dt, int root, ReductionOp op) override {
    BAGUA_NCCL_CHECK(ncclReduce(send, recv, (size_t)count, to_nccl(dt), to_nccl(op), root, comm_, stream_));
  }
  void send(const void* buf, int64_t count, DType dt, int peer) override {
    BAGUA_NCCL_CHECK(ncclSend(buf, (size_t)count, to_nccl(dt), peer, comm_, stream_));
  }
  void recv(void* buf, int64_t count, DType dt, int peer) override {
    BAGUA_NCCL_CHECK(ncclRecv(buf, (size_t)count, to_nccl(dt), peer, comm_, stream_));
  }
  void alltoall(const void* send, void* recv, int64_t count, DType dt) override {
    const size_t es = dtype_bytes(dt);
    BAGUA_NCCL_CHECK(ncclGroupStart());
    for (int p = 0; p < nranks_; ++p) {
      BAGUA_NCCL_CHECK(ncclSend((const char*)send + (size_t)p * count * es, (size_t)count, to_nccl(dt), p, comm_, stream_));
      BAGUA_NCCL_CHECK(ncclRecv((char*)recv + (size_t)p * count * es, (size_t)count, to_nccl(dt), p, comm_, stream_));
    }
    BAGUA_NCCL_CHECK(ncclGroupEnd());
  }
  void alltoall_v(const void* send, const std::vector<int64_t>& sc, const std::vector<int64_t>& sd, void* recv,
                  const std::vector<int64_t>& rc, const std::vector<int64_t>& rd, DType dt) override {
    const size_t es = dtype_bytes(dt);
    BAGUA_NCCL_CHECK(ncclGroupStart());
    for (int p = 0; p < nranks_; ++p) {
      if (sc[p] > 0)
        BAGUA_NCCL_CHECK(ncclSend((const char*)send + (size_t)sd[p] * es, (size_t)sc[p], to_nccl(dt), p, comm_, stream_));
      if (rc[p] > 0)
        BAGUA_NCCL_CHECK(ncclRecv((char*)recv + (size_t)rd[p] * es, (size_t)rc[p], to_nccl(dt), p, comm_, stream_));
    }
    BAGUA_NCCL_CHECK(ncclGroupEnd());
  }
  void allgather(const void* send, void* recv, int64_t count, DType dt) override {
    BAGUA_NCCL_CHECK(ncclAllGather(send, recv, (size_t)count, to_nccl(dt), comm_, stream_));
  }
  void gather(const void* send, void* recv, int64_t count, DType dt, int root) override {
    const size_t es = dtype_bytes(dt);
    BAGUA_NCCL_CHECK(ncclGroupStart());
    BAGUA_NCCL_CHECK(ncclSend(send, (size_t)count, to_nccl(dt), root, comm_, stream_));
    if (rank_ == root)
      for (int p = 0; p < nranks_; ++p)
        BAGUA_NCCL_CHECK(ncclRecv((char*)recv + (size_t)p * count * es, (size_t)count, to_nccl(dt), p, comm_, stream_));
    BAGUA_NCCL_CHECK(ncclGroupEnd());
  }
  void scatter(const void* send, void* recv, int64_t count, DType dt, int root) override {
    const size_t es = dtype_bytes(dt);
    BAGUA_NCCL_CHECK(ncclGroupStart());
    if (rank_ == root)
      for (int p = 0; p < nranks_; ++p)
        BAGUA_NCCL_CHECK(ncclSend((const char*)send + (size_t)p * count * es, (size_t)count, to_nccl(dt), p, comm_, stream_));
    BAGUA_NCCL_CHECK(ncclRecv(recv, (size_t)count, to_nccl(dt), root, comm_, stream_));
    BAGUA_NCCL_CHECK(ncclGroupEnd());
  }
  void reduce_scatter(const void* send, void* recv, int64_t recv_count, DType dt, ReductionOp op) override {
    BAGUA_NCCL_CHECK(ncclReduceScatter(send, recv, (size_t)recv_count, to_nccl(dt), to_nccl(op), comm_, stream_));
  }
  void barrier() override {
    // NCCL has no barrier: all-reduce one word and wait for it on the host.
    if (!barrier_buf_) BAGUA_CUDA_CHECK(cudaMalloc(&barrier_buf_, 256));
    BAGUA_NCCL_CHECK(ncclAllReduce(barrier_buf_, barrier_buf_, 1, ncclFloat32, ncclSum, comm_, stream_));
    BAGUA_CUDA_CHECK(cudaStreamSynchronize(stream_));
  }
  void group_start() override { BAGUA_NCCL_CHECK(ncclGroupStart()); }
  void group_end() override { BAGUA_NCCL_CHECK(ncclGroupEnd()); }
  void abort() override {
    if (comm_) {
      ncclCommAbort(comm_);
      comm_ = nullptr;
    }
  }

 private:
  int rank_, nranks_, device_;
  cudaStream_t stream_;
  ncclComm_t comm_ = nullptr;
  void* barrier_buf_ = nullptr;
};

}  // namespace

std::unique_ptr<Transport> make_nccl_transport(int rank, int nranks, int device_id, uint64_t stream,
                                               const std::string& unique_id_b64) {
  return std::make_unique<NcclTransport>(rank, nranks, device_id, stream, unique_id_b64);
}

std::string nccl_generate_unique_id_b64() {
  ncclUniqueId id;
  BAGUA_NCCL_CHECK(ncclGetUniqueId(&id));
  return base64_encode(std::string((const char*)&id, sizeof(id)));
}

int nccl_version() {
  int v = 0;
  if (ncclGetVersion(&v) != ncclSuccess) return 0;
  return v;
}

}  // namespace bagua
