// Library collective transport behind a communicator.
//
// Two implementations: NCCL on a CUDA stream (bootstrap of the peer arena, the measured
// baseline path, and the fallback for layouts the fused kernels do not take) and c10d
// (gloo) on host memory, which is what the CPU backend and the multi-process CPU tests
// use.  The reference reaches NCCL through Aluminum
// (bagua-core-internal/src/communicators/mod.rs:473-1043).
#pragma once

#include "../common.h"

namespace bagua {

class Transport {
 public:
  virtual ~Transport() = default;
  virtual int rank() const = 0;
  virtual int nranks() const = 0;
  virtual const char* kind() const = 0;

  virtual void allreduce(const void* send, void* recv, int64_t count, DType dt, ReductionOp op) = 0;
  virtual void broadcast(void* buf, int64_t count, DType dt, int root) = 0;
  virtual void reduce(const void* send, void* recv, int64_t count, DType dt, int root, ReductionOp op) = 0;
  virtual void send(const void* buf, int64_t count, DType dt, int peer) = 0;
  virtual void recv(void* buf, int64_t count, DType dt, int peer) = 0;
  // equal split: `count` elements to/from every rank; send and recv must not alias
  virtual void alltoall(const void* send, void* recv, int64_t count, DType dt) = 0;
  virtual void alltoall_v(const void* send, const std::vector<int64_t>& send_counts,
                          const std::vector<int64_t>& send_displs, void* recv,
                          const std::vector<int64_t>& recv_counts, const std::vector<int64_t>& recv_displs,
                          DType dt) = 0;
  // recv holds nranks*count; `send` may alias its own slot
  virtual void allgather(const void* send, void* recv, int64_t count, DType dt) = 0;
  virtual void gather(const void* send, void* recv, int64_t count, DType dt, int root) = 0;
  virtual void scatter(const void* send, void* recv, int64_t count, DType dt, int root) = 0;
  // send holds nranks*recv_count
  virtual void reduce_scatter(const void* send, void* recv, int64_t recv_count, DType dt, ReductionOp op) = 0;
  virtual void barrier() = 0;
  virtual void group_start() = 0;
  virtual void group_end() = 0;
  virtual void abort() = 0;
};

// Defined in nccl_transport.cc.
std::unique_ptr<Transport> make_nccl_transport(int rank, int nranks, int device_id, uint64_t stream,
                                               const std::string& unique_id_b64);
std::string nccl_generate_unique_id_b64();
int nccl_version();

// Defined in c10d_transport.cc: wraps the process group registered under `group_name`
// in this process (see torch.distributed `ProcessGroup.group_name`).
std::unique_ptr<Transport> make_c10d_transport(int rank, int nranks, const std::string& group_name);

// Defined in solo_transport.cc: a communicator of one rank (unique id "solo"), on device memory
// (stream-ordered copies) or, with device_id < 0, on host memory.
std::unique_ptr<Transport> make_solo_transport(int device_id, uint64_t stream);
inline bool is_solo_unique_id(const std::string& s) { return s == "solo"; }

// Unique-id strings of the form "c10d:<group name>" select the c10d transport.
inline bool is_c10d_unique_id(const std::string& s) { return s.rfind("c10d:", 0) == 0; }

}  // namespace bagua
