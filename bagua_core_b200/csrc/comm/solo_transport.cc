// The one-rank transport: every collective over a single rank is a copy or nothing.
//
// Used for the "inter-node" tier of a hierarchical communicator whose node is the whole job
// (one NVSwitch box): the reference runs that tier on the leader through an NCCL communicator
// of one rank and broadcasts the result (bagua-core-internal/src/communicators/mod.rs:390-427);
// here every rank runs the tier's (deterministic) work on its own copy of the reduced bucket,
// which gives the same bits without the broadcast.  Unique id "solo".
#include <cuda_runtime.h>

#include <cstring>

#include "transport.h"

namespace bagua {

namespace {

class SoloTransport : public Transport {
 public:
  SoloTransport(int device, uint64_t stream) : device_(device), stream_((cudaStream_t)stream) {}
  int rank() const override { return 0; }
  int nranks() const override { return 1; }
  const char* kind() const override { return "solo"; }

  void allreduce(const void* send, void* recv, int64_t count, DType dt, ReductionOp) override {
    copy(recv, send, count, dt);  // sum, mean, min, max ... of one value is the value
  }
  void broadcast(void*, int64_t, DType, int root) override { need_self(root); }
  void reduce(const void* send, void* recv, int64_t count, DType dt, int root, ReductionOp) override {
    need_self(root);
    copy(recv, send, count, dt);
  }
  void send(const void*, int64_t, DType, int) override { no_peer(); }
  void recv(void*, int64_t, DType, int) override { no_peer(); }
  void alltoall(const void* send, void* recv, int64_t count, DType dt) override { copy(recv, send, count, dt); }
  void alltoall_v(const void* send, const std::vector<int64_t>& sc, const std::vector<int64_t>& sd, void* recv,
                  const std::vector<int64_t>& rc, const std::vector<int64_t>& rd, DType dt) override {
    BAGUA_CHECK(sc.size() == 1 && rc.size() == 1 && sc[0] == rc[0], Communicator,
                "alltoall_v over one rank: send and recv counts must agree");
    const size_t es = dtype_bytes(dt);
    copy((char*)recv + (size_t)rd[0] * es, (const char*)send + (size_t)sd[0] * es, sc[0], dt);
  }
  void allgather(const void* send, void* recv, int64_t count, DType dt) override { copy(recv, send, count, dt); }
  void gather(const void* send, void* recv, int64_t count, DType dt, int root) override {
    need_self(root);
    copy(recv, send, count, dt);
  }
  void scatter(const void* send, void* recv, int64_t count, DType dt, int root) override {
    need_self(root);
    copy(recv, send, count, dt);
  }
  void reduce_scatter(const void* send, void* recv, int64_t recv_count, DType dt, ReductionOp) override {
    copy(recv, send, recv_count, dt);
  }
  void barrier() override {
    if (device_ >= 0) BAGUA_CUDA_CHECK(cudaStreamSynchronize(stream_));
  }
  void group_start() override {}
  void group_end() override {}
  void abort() override {}

 private:
  void copy(void* dst, const void* src, int64_t count, DType dt) {
    if (dst == src || count <= 0) return;
    const size_t bytes = (size_t)count * dtype_bytes(dt);
    if (device_ >= 0)
      BAGUA_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream_));
    else
      std::memmove(dst, src, bytes);
  }
  static void need_self(int root) {
    BAGUA_CHECK(root == 0, Communicator, "a communicator of one rank has no rank " << root);
  }
  [[noreturn]] static void no_peer() {
    throw BaguaError(ErrorKind::Communicator, "send / recv on a communicator of one rank: there is no peer");
  }
  int device_;
  cudaStream_t stream_;
};

}  // namespace

std::unique_ptr<Transport> make_solo_transport(int device_id, uint64_t stream) {
  return std::make_unique<SoloTransport>(device_id, stream);
}

}  // namespace bagua
