// Python bindings (pybind11): the `bagua_core` API surface plus the hooks the
// `bagua_core_b200` Python layer and the tests use.
//
// Reference surface: bagua-core-py/src/lib.rs:21-193 (BaguaSingleCommunicatorPy),
// 203-298 (BaguaTensorPy), 308-349 (BaguaCommBackendPy), 359-485 (BaguaBucketPy),
// 506-514 (module).  Method names, argument order, defaults and the `op: u8` encoding
// are kept.  Blocking calls release the GIL; every BaguaError surfaces as RuntimeError.
// Tensor metadata comes from `at::Tensor`'s public API instead of private struct
// layouts (bagua-core-internal/src/torch_ffi.rs).
#include <cuda_runtime.h>
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "comm/arena.h"
#include "comm/communicator.h"
#include "kernels/fused.h"
#include "kernels/fused_emu.h"
#include "kernels/kernels.h"
#include "kernels/model_ops.h"
#include "ops/comm_op.h"
#include "pool/resource_pool.h"
#include "runtime/backend.h"
#include "runtime/timeline.h"
#include "telemetry/telemetry.h"
#include "tensor/tensor.h"

namespace py = pybind11;
using namespace bagua;

namespace {

DType dtype_from_torch(at::ScalarType st) {
  switch (st) {
    case at::kFloat: return DType::F32;
    case at::kHalf: return DType::F16;
    case at::kLong: return DType::I64;
    case at::kByte: return DType::U8;
    case at::kBFloat16: return DType::BF16;
    default: throw BaguaError(ErrorKind::Tensor, std::string("unsupported tensor dtype ") + c10::toString(st));
  }
}

// A framework tensor: every query goes to the live at::Tensor, so storage swaps made by
// the Python layer (flattening into bucket storage) are seen without re-registration.
class TorchRawTensor : public RawTensor {
 public:
  explicit TorchRawTensor(at::Tensor t) : t_(std::move(t)), dtype_(dtype_from_torch(t_.scalar_type())) {
    BAGUA_CHECK(t_.is_non_overlapping_and_dense(), Tensor, "bagua tensors must be dense (no gaps, no overlap)");
    BAGUA_CHECK(t_.is_cuda() || t_.is_cpu(), Tensor, "bagua tensors must live on a CUDA device or on the host");
  }
  ~TorchRawTensor() override {
    // at::Tensor may hold the last reference to Python-owned memory.
    py::gil_scoped_acquire g;
    t_.reset();
  }
  void* data_ptr() const override { return t_.data_ptr(); }
  int64_t num_elements() const override { return t_.numel(); }
  int64_t num_elements_allocated() const override { return t_.numel(); }
  int device_id() const override { return t_.is_cuda() ? (int)t_.device().index() : -1; }
  DType dtype() const override { return dtype_; }
  const at::Tensor& tensor() const { return t_; }

 private:
  at::Tensor t_;
  DType dtype_;
};

struct PyTensor {
  TensorPtr inner;
};
struct PyBucket {
  BucketPtr inner;
  std::vector<py::object> py_tensors;  // keeps the Python wrappers alive for tensors()
};
struct PyComm {
  SingleCommPtr inner;
};
struct PyBackend {
  std::unique_ptr<CommBackend> inner;
};

SingleCommPtr opt_comm(const py::object& o) { return o.is_none() ? nullptr : o.cast<PyComm&>().inner; }

kernels::Ctx ctx_of(const at::Tensor& t, uint64_t stream) {
  return kernels::Ctx{t.is_cuda() ? (int)t.device().index() : -1, (cudaStream_t)stream};
}

void check_pair(const at::Tensor& a, const at::Tensor& b) {
  BAGUA_CHECK(a.scalar_type() == b.scalar_type() && a.numel() == b.numel() && a.device() == b.device() &&
                  a.is_contiguous() && b.is_contiguous(),
              Tensor, "tensors must be contiguous and agree in dtype, size and device");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "bagua-core for B200: scheduler, buckets, communicators and fused sm_100a communication kernels";

  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const BaguaError& e) {
      PyErr_SetString(PyExc_RuntimeError, e.what());
    }
  });

  // -------------------------------------------------------------------------------
  py::class_<PyComm>(m, "BaguaSingleCommunicatorPy", py::dynamic_attr())
      .def(py::init([](int rank, int nranks, int device_id, uint64_t stream_ptr, const std::string& uid) {
             py::gil_scoped_release rel;
             return PyComm{std::make_shared<SingleCommunicator>(rank, nranks, device_id, stream_ptr, uid)};
           }),
           py::arg("rank"), py::arg("nranks"), py::arg("device_id"), py::arg("stream_ptr"),
           py::arg("nccl_unique_id_str"))
      .def("nranks", [](PyComm& c) { return c.inner->nranks(); })
      .def("rank", [](PyComm& c) { return c.inner->rank(); })
      .def("device_id", [](PyComm& c) { return c.inner->device_id(); })
      .def("abort", [](PyComm& c) { c.inner->abort(); }, py::call_guard<py::gil_scoped_release>())
      .def("check_abort", [](PyComm& c) { return c.inner->check_abort(); })
      .def("allreduce",
           [](PyComm& c, PyTensor& s, PyTensor& r, int op) {
             c.inner->allreduce(*s.inner->raw(), *r.inner->raw(), reduction_op_from_u8(op));
           },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("op"), py::call_guard<py::gil_scoped_release>())
      .def("allreduce_inplace",
           [](PyComm& c, PyTensor& t, int op) { c.inner->allreduce_inplace(*t.inner->raw(), reduction_op_from_u8(op)); },
           py::arg("tensor"), py::arg("op"), py::call_guard<py::gil_scoped_release>())
      .def("broadcast", [](PyComm& c, PyTensor& t, int root) { c.inner->broadcast(*t.inner->raw(), root); },
           py::arg("tensor"), py::arg("root_rank"), py::call_guard<py::gil_scoped_release>())
      .def("reduce",
           [](PyComm& c, PyTensor& s, PyTensor& r, int dst, int op) {
             c.inner->reduce(*s.inner->raw(), *r.inner->raw(), dst, reduction_op_from_u8(op));
           },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("dst"), py::arg("op"),
           py::call_guard<py::gil_scoped_release>())
      .def("reduce_inplace",
           [](PyComm& c, PyTensor& t, int dst, int op) {
             c.inner->reduce_inplace(*t.inner->raw(), dst, reduction_op_from_u8(op));
           },
           py::arg("tensor"), py::arg("dst"), py::arg("op"), py::call_guard<py::gil_scoped_release>())
      .def("send", [](PyComm& c, PyTensor& t, int peer) { c.inner->send(*t.inner->raw(), peer); }, py::arg("tensor"),
           py::arg("peer_rank"), py::call_guard<py::gil_scoped_release>())
      .def("recv", [](PyComm& c, PyTensor& t, int peer) { c.inner->recv(*t.inner->raw(), peer); }, py::arg("tensor"),
           py::arg("peer_rank"), py::call_guard<py::gil_scoped_release>())
      .def("alltoall", [](PyComm& c, PyTensor& s, PyTensor& r) { c.inner->alltoall(*s.inner->raw(), *r.inner->raw()); },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::call_guard<py::gil_scoped_release>())
      .def("alltoall_inplace", [](PyComm& c, PyTensor& t) { c.inner->alltoall_inplace(*t.inner->raw()); },
           py::arg("tensor"), py::call_guard<py::gil_scoped_release>())
      .def("alltoall_v",
           [](PyComm& c, PyTensor& s, std::vector<int64_t> sc, std::vector<int64_t> sd, PyTensor& r,
              std::vector<int64_t> rc, std::vector<int64_t> rd) {
             c.inner->alltoall_v(*s.inner->raw(), sc, sd, *r.inner->raw(), rc, rd);
           },
           py::arg("send_tensor"), py::arg("send_counts"), py::arg("send_displs"), py::arg("recv_tensor"),
           py::arg("recv_counts"), py::arg("recv_displs"), py::call_guard<py::gil_scoped_release>())
      .def("allgather",
           [](PyComm& c, PyTensor& s, PyTensor& r) { c.inner->allgather(*s.inner->raw(), *r.inner->raw()); },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::call_guard<py::gil_scoped_release>())
      .def("allgather_inplace", [](PyComm& c, PyTensor& t) { c.inner->allgather_inplace(*t.inner->raw()); },
           py::arg("tensor"), py::call_guard<py::gil_scoped_release>())
      .def("gather",
           [](PyComm& c, PyTensor& s, PyTensor& r, int dst) { c.inner->gather(*s.inner->raw(), *r.inner->raw(), dst); },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("dst"), py::call_guard<py::gil_scoped_release>())
      .def("gather_inplace",
           [](PyComm& c, PyTensor& t, int64_t count, int dst) { c.inner->gather_inplace(*t.inner->raw(), count, dst); },
           py::arg("tensor"), py::arg("count"), py::arg("dst"), py::call_guard<py::gil_scoped_release>())
      .def("scatter",
           [](PyComm& c, PyTensor& s, PyTensor& r, int src) { c.inner->scatter(*s.inner->raw(), *r.inner->raw(), src); },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("src"), py::call_guard<py::gil_scoped_release>())
      .def("scatter_inplace",
           [](PyComm& c, PyTensor& t, int64_t count, int src) {
             c.inner->scatter_inplace(*t.inner->raw(), count, src);
           },
           py::arg("tensor"), py::arg("count"), py::arg("src"), py::call_guard<py::gil_scoped_release>())
      .def("reduce_scatter",
           [](PyComm& c, PyTensor& s, PyTensor& r, int op) {
             c.inner->reduce_scatter(*s.inner->raw(), *r.inner->raw(), reduction_op_from_u8(op));
           },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("op"), py::call_guard<py::gil_scoped_release>())
      .def("reduce_scatter_inplace",
           [](PyComm& c, PyTensor& t, int op) {
             c.inner->reduce_scatter_inplace(*t.inner->raw(), reduction_op_from_u8(op));
           },
           py::arg("tensor"), py::arg("op"), py::call_guard<py::gil_scoped_release>())
      .def("barrier", [](PyComm& c) { c.inner->barrier(); }, py::call_guard<py::gil_scoped_release>())
      .def_static("generate_nccl_unique_id_str", []() { return nccl_generate_unique_id_b64(); })
      // ---- additions for the B200 engine ----
      .def("transport", [](PyComm& c) { return std::string(c.inner->transport_kind()); })
      .def("set_fused", [](PyComm& c, bool on) { c.inner->set_fused(on); },
           "Enable/disable the fused peer-memory kernels for ops on this communicator.")
      .def("set_p2p_collectives", [](PyComm& c, bool on) { c.inner->set_p2p_collectives(on); },
           "Run this communicator's own collectives (allreduce / reduce / reduce_scatter with SUM or AVG, allgather, "
           "alltoall, gather, scatter, broadcast, barrier) as peer-memory kernels instead of library calls (also BAGUA_B200_P2P_COLLECTIVES=1). "
           "Must be set identically on every rank.")
      .def("p2p_collectives", [](PyComm& c) { return c.inner->p2p_collectives(); })
      .def("fused_available", [](PyComm& c) { return c.inner->arena() != nullptr; },
           py::call_guard<py::gil_scoped_release>(),
           "Collective: sets up the peer arena if needed and reports whether fused kernels can be used.")
      .def("set_device_wait_ms",
           [](PyComm& c, double ms) {
             if (auto* a = c.inner->arena()) a->set_deadline_ms(ms);
           },
           py::call_guard<py::gil_scoped_release>())
      .def("check_device_status", [](PyComm& c) { c.inner->check_device_status(); })
      .def("set_comm_ctas",
           [](PyComm& c, int ctas, int coop_ctas) {
             if (auto* a = c.inner->arena()) {
               if (ctas > 0) a->set_max_blocks(ctas);
               if (coop_ctas > 0) a->set_max_coop_blocks(coop_ctas);
             }
           },
           py::arg("ctas"), py::arg("coop_ctas") = 0, py::call_guard<py::gil_scoped_release>(),
           "CTA budgets of this communicator's fused kernels (BAGUA_B200_COMM_CTAS / BAGUA_B200_COOP_CTAS); "
           "0 leaves one unchanged.  Must be set identically on every rank.")
      .def(
          "alloc_symmetric",
          [](PyComm& c, int64_t numel, at::ScalarType dtype) -> py::object {
            PeerArena* a = nullptr;
            void* ptr = nullptr;
            const size_t bytes = (size_t)numel * c10::elementSize(dtype);
            {
              py::gil_scoped_release rel;
              a = c.inner->arena();
              if (a) ptr = a->sym_alloc(bytes);
            }
            if (!a) return py::none();
            // the memory belongs to the communicator's arena: keep the communicator alive
            // for as long as any tensor views it
            SingleCommPtr keep = c.inner;
            at::Tensor t = at::from_blob(
                ptr, {numel}, [keep](void*) {},
                at::TensorOptions().dtype(dtype).device(at::kCUDA, c.inner->device_id()));
            return py::cast(t);
          },
          py::arg("numel"), py::arg("dtype"),
          "Collective: a 1-D CUDA tensor in memory that every rank of this communicator maps (all ranks must "
          "call with the same sizes in the same order).  Buckets placed here are all-reduced in place without "
          "staging copies.  Returns None when the peer arena is not available.")
      .def("is_symmetric",
           [](PyComm& c, const at::Tensor& t) {
             PeerArena* a = c.inner->arena();
             void* peers[kArenaMaxRanks];
             return a && t.is_cuda() && a->sym_translate(t.data_ptr(), t.nbytes(), peers);
           })
      .def("is_nvls_mapped",
           [](PyComm& c, const at::Tensor& t) {
             PeerArena* a = c.inner->arena();
             return a && t.is_cuda() && a->sym_multicast(t.data_ptr(), t.nbytes()) != nullptr;
           },
           "True if the tensor lies in symmetric memory that also has an NVSwitch multicast mapping "
           "(BAGUA_B200_NVLS=1 on a platform that supports it): its all-reduce runs inside the switch.")
      .def("fused_launches", [](PyComm& c) {
        auto* a = c.inner->arena();
        return a ? a->fused_launches() : (uint64_t)0;
      })
      .def("fused_allreduce_ce",
           [](PyComm& c, PyTensor& s, PyTensor& r, bool average) {
             auto* a = c.inner->arena();
             BAGUA_CHECK(a != nullptr, Communicator, "fused kernels are not available on this communicator");
             auto sr = s.inner->raw();
             auto rr = r.inner->raw();
             BAGUA_CHECK(sr->dtype() == rr->dtype() && sr->num_elements_allocated() == rr->num_elements_allocated(),
                         Tensor, "send and recv must agree in dtype and size");
             return fused::allreduce_ce(*a, sr->data_ptr(), rr->data_ptr(), sr->num_elements_allocated(), sr->dtype(),
                                        average ? 1.0f / (float)c.inner->nranks() : 1.0f,
                                        (cudaStream_t)c.inner->stream());
           },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("average"),
           py::call_guard<py::gil_scoped_release>(),
           "All-reduce of symmetric buffers with the bytes moved by the copy engines (False: not symmetric).")
      .def("fused_allreduce",
           [](PyComm& c, PyTensor& s, PyTensor& r, bool average) {
             auto* a = c.inner->arena();
             BAGUA_CHECK(a != nullptr, Communicator, "fused kernels are not available on this communicator");
             auto sr = s.inner->raw();
             auto rr = r.inner->raw();
             BAGUA_CHECK(sr->dtype() == rr->dtype() && sr->num_elements_allocated() == rr->num_elements_allocated(),
                         Tensor, "send and recv must agree in dtype and size");
             return fused::allreduce(*a, sr->data_ptr(), rr->data_ptr(), sr->num_elements_allocated(), sr->dtype(),
                                     average ? 1.0f / (float)c.inner->nranks() : 1.0f, (cudaStream_t)c.inner->stream());
           },
           py::arg("send_tensor"), py::arg("recv_tensor"), py::arg("average"),
           py::call_guard<py::gil_scoped_release>(),
           "Launch the fused all-reduce kernel directly (returns False if the layout is not eligible).");

  // -------------------------------------------------------------------------------
  py::class_<PyTensor>(m, "BaguaTensorPy", py::dynamic_attr())
      .def(py::init([](const at::Tensor& t, const std::string& name) {
             return PyTensor{std::make_shared<BaguaTensor>(name, std::make_shared<TorchRawTensor>(t))};
           }),
           py::arg("torch_tensor"), py::arg("name"))
      .def("compress",
           [](PyTensor& t, const std::string& method, int n_chunks, int target_chunk) {
             return PyTensor{t.inner->compress(method, n_chunks, target_chunk)};
           },
           py::arg("method"), py::arg("n_chunks"), py::arg("target_chunk"), py::call_guard<py::gil_scoped_release>())
      .def("decompress_from",
           [](PyTensor& t, const std::string& method, int n_chunks, PyTensor& c) {
             t.inner->decompress_from(method, n_chunks, *c.inner);
           },
           py::arg("method"), py::arg("n_chunks"), py::arg("compressed_buffer"),
           py::call_guard<py::gil_scoped_release>())
      .def("to_numpy_f32",
           [](PyTensor& t) {
             BAGUA_CHECK(t.inner->dtype() == DType::F32, Tensor, "to_numpy_f32 needs an F32 tensor");
             py::array_t<float> a((py::ssize_t)t.inner->num_elements());
             t.inner->copy_to_host(a.mutable_data());
             return a;
           })
      .def("to_numpy_u8",
           [](PyTensor& t) {
             BAGUA_CHECK(t.inner->dtype() == DType::U8, Tensor, "to_numpy_u8 needs a U8 tensor");
             py::array_t<uint8_t> a((py::ssize_t)t.inner->num_elements());
             t.inner->copy_to_host(a.mutable_data());
             return a;
           })
      .def("data_ptr", [](PyTensor& t) { return t.inner->data_ptr(); })
      .def("device_id", [](PyTensor& t) { return t.inner->device_id(); })
      .def("num_elements", [](PyTensor& t) { return t.inner->num_elements(); })
      .def("num_elements_allocated", [](PyTensor& t) { return t.inner->num_elements_allocated(); })
      .def("dtype", [](PyTensor& t) { return std::string(dtype_name(t.inner->dtype())); })
      .def("name", [](PyTensor& t) { return t.inner->name(); })
      .def("ready_for_comm", [](PyTensor& t) { return t.inner->ready_for_comm(); })
      .def("torch_tensor", [](PyTensor& t) -> py::object {
        auto raw = t.inner->raw();
        if (auto* tr = dynamic_cast<TorchRawTensor*>(raw.get())) return py::cast(tr->tensor());
        return py::none();
      });

  // -------------------------------------------------------------------------------
  py::class_<PyBucket>(m, "BaguaBucketPy", py::dynamic_attr())
      .def(py::init([](const std::string& name, py::list tensors) {
             PyBucket b;
             std::vector<TensorPtr> ts;
             for (auto h : tensors) {
               ts.push_back(h.cast<PyTensor&>().inner);
               b.py_tensors.push_back(py::reinterpret_borrow<py::object>(h));
             }
             b.inner = std::make_shared<BaguaBucket>(name, std::move(ts));
             return b;
           }),
           py::arg("name"), py::arg("tensors"))
      .def("tensors", [](PyBucket& b) { return b.py_tensors; })
      .def("name", [](PyBucket& b) { return b.inner->name(); })
      .def("append_python_op",
           [](PyBucket& b, py::object op) {
             if (!PyCallable_Check(op.ptr())) throw py::type_error("python op should be a callable");
             // the callable is released under the GIL, whichever thread drops the op
             auto holder = std::shared_ptr<py::object>(new py::object(std::move(op)), [](py::object* o) {
               py::gil_scoped_acquire g;
               delete o;
             });
             b.inner->append_op(make_callback_op(
                 [holder](const std::string& bucket_name) {
                   py::gil_scoped_acquire g;
                   try {
                     (*holder)(bucket_name);
                   } catch (py::error_already_set& e) {
                     std::string what = e.what();
                     e.restore();
                     PyErr_Clear();
                     throw std::runtime_error(what);
                   }
                 },
                 "python callable"));
           },
           py::arg("op"))
      .def("append_centralized_synchronous_op",
           [](PyBucket& b, py::object inter, py::object intra, bool hierarchical, bool average, bool scattergather,
              py::object compression) {
             auto comm = Communicator::create(opt_comm(inter), opt_comm(intra), hierarchical);
             if (compression.is_none())
               b.inner->append_op(make_centralized_full_precision_op(comm, average, scattergather));
             else
               b.inner->append_op(make_centralized_low_precision_op(comm, average, compression.cast<std::string>()));
           },
           py::arg("communicator_internode") = py::none(), py::arg("communicator_intranode") = py::none(),
           py::arg("hierarchical") = false, py::arg("average") = true, py::arg("scattergather") = false,
           py::arg("compression") = py::none())
      .def("append_decentralized_synchronous_op",
           [](PyBucket& b, py::object inter, py::object intra, bool hierarchical, const std::string& mode,
              PyTensor& peer_weight) {
             auto comm = Communicator::create(opt_comm(inter), opt_comm(intra), hierarchical);
             b.inner->append_op(
                 make_decentralized_full_precision_op(comm, parse_peer_selection_mode(mode), peer_weight.inner));
           },
           py::arg("communicator_internode") = py::none(), py::arg("communicator_intranode") = py::none(),
           py::arg("hierarchical") = false, py::arg("peer_selection_mode"), py::arg("peer_weight"))
      .def("append_low_precision_decentralized_synchronous_op",
           [](PyBucket& b, py::object inter, py::object intra, bool hierarchical, const std::string& mode,
              const std::string& compression, PyTensor& w, PyTensor& l, PyTensor& r) {
             auto comm = Communicator::create(opt_comm(inter), opt_comm(intra), hierarchical);
             b.inner->append_op(make_decentralized_low_precision_op(comm, parse_peer_selection_mode(mode), compression,
                                                                    w.inner, l.inner, r.inner));
           },
           py::arg("communicator_internode") = py::none(), py::arg("communicator_intranode") = py::none(),
           py::arg("hierarchical") = false, py::arg("peer_selection_mode"), py::arg("compression"), py::arg("weight"),
           py::arg("left_peer_weight"), py::arg("right_peer_weight"))
      .def("append_decentralized_asynchronous_op",
           [](PyBucket& b, py::object inter, py::object intra, const std::string& mode, uint64_t torch_stream) {
             auto comm = Communicator::create(opt_comm(inter), opt_comm(intra), false);
             b.inner->append_op(make_decentralized_async_op(comm, parse_peer_selection_mode(mode), torch_stream));
           },
           py::arg("communicator_internode") = py::none(), py::arg("communicator_intranode") = py::none(),
           py::arg("peer_selection_mode"), py::arg("torch_stream"))
      .def("print_ops", [](PyBucket& b) { py::print(b.inner->describe_ops()); })
      .def("describe_ops", [](PyBucket& b) { return b.inner->describe_ops(); })
      .def("clear_ops", [](PyBucket& b) { b.inner->clear_ops(); })
      .def("ready_for_comm", [](PyBucket& b) { return b.inner->ready_for_comm(); })
      .def("reset_comm_ready", [](PyBucket& b) { b.inner->reset_comm_ready(); })
      .def("ops_state",
           [](PyBucket& b) {
             std::vector<std::vector<std::pair<std::string, int64_t>>> out;
             for (auto& o : b.inner->ops_snapshot()) out.push_back(o->state());
             return out;
           },
           "Checkpointable state of every op of the bucket (e.g. the gossip step counter).")
      .def("load_ops_state", [](PyBucket& b, std::vector<std::vector<std::pair<std::string, int64_t>>> st) {
        auto ops = b.inner->ops_snapshot();
        BAGUA_CHECK(st.size() == ops.size(), Bucket, "state does not match the bucket's ops");
        for (size_t i = 0; i < ops.size(); ++i) ops[i]->load_state(st[i]);
      });

  // -------------------------------------------------------------------------------
  py::class_<PyBackend>(m, "BaguaCommBackendPy", py::dynamic_attr())
      .def(py::init([](size_t cap, int device_id) {
             return PyBackend{std::make_unique<CommBackend>(cap, device_id)};
           }),
           py::arg("schedule_channel_cap"), py::arg("device_id"))
      .def("register_ordered_buckets",
           [](PyBackend& be, py::list buckets) {
             std::vector<BucketPtr> bs;
             for (auto h : buckets) bs.push_back(h.cast<PyBucket&>().inner);
             py::gil_scoped_release rel;
             be.inner->register_ordered_buckets(bs);
           },
           py::arg("buckets"))
      .def("mark_communication_ready",
           [](PyBackend& be, PyTensor& t, uint64_t ev) { be.inner->mark_communication_ready(t.inner, ev); },
           py::arg("tensor"), py::arg("ready_cuda_event_ptr"), py::call_guard<py::gil_scoped_release>())
      .def("wait_pending_comm_ops", [](PyBackend& be) { return be.inner->wait_pending_comm_ops(); },
           py::call_guard<py::gil_scoped_release>())
      .def("set_watchdog_timeout", [](PyBackend& be, double s) { be.inner->set_watchdog_timeout(s); })
      .def("watchdog_timeout", [](PyBackend& be) { return be.inner->watchdog_timeout(); })
      .def("pending", [](PyBackend& be) { return be.inner->pending(); },
           "Scheduled buckets whose completion nobody has waited for yet.")
      .def("close", [](PyBackend& be) {
        py::gil_scoped_release rel;
        be.inner.reset();
      });

  // -------------------------------------------------------------------------------
  m.def("show_version", []() {
    std::fprintf(stderr, "project_name: bagua-core-b200\nis_debug: false\nversion: %s\n", "0.1.0");
    std::fprintf(stderr, "build: %s %s, nvcc target sm_100a\n", __DATE__, __TIME__);
    int rt = 0;
    cudaRuntimeGetVersion(&rt);
    std::fprintf(stderr, "cuda runtime: %d\nNCCL version: %d\n", rt, nccl_version());
  });
  m.def("nccl_version", &nccl_version);

  // engine configuration / statistics
  m.def("set_sync_per_bucket", [](bool on) { EngineConfig::global().sync_per_bucket = on; },
        "Reference-faithful mode: synchronise the communication stream after every bucket.");
  m.def("get_sync_per_bucket", []() { return EngineConfig::global().sync_per_bucket; });
  m.def(
      "set_tuning",
      [](const std::string& key, long value) {
        BAGUA_CHECK(fused::Tuning::global().set(key, value), Backend, "unknown tuning key `" << key << "`");
      },
      py::arg("key"), py::arg("value"),
      "Size thresholds and CTA budgets of the fused kernels (keys: oneshot_bytes, oneshot_sym_bytes, overlap_ctas, "
      "nvls_overlap_ctas, coop_overlap_ctas, bytes_per_cta, sym_threads, pair_sym_min_bytes, ce_min_bytes, ce_min_chunk_bytes, tma_min_bytes, tma_isolated, tma_ctas, "
      "tma_overlap_ctas, tma_bytes_per_cta; defaults from BAGUA_B200_<KEY>).  Must be set identically on every rank.");
  m.def("get_tuning", []() {
    py::dict d;
    for (auto& kv : fused::Tuning::global().items()) d[py::str(kv.first)] = kv.second;
    return d;
  });
  m.def("set_bucket_timing", [](bool on) { BucketTimeline::instance().set_enabled(on); }, py::arg("on"),
        "Record two timing events per bucket on the communication stream (also BAGUA_B200_BUCKET_TIMING=1).");
  m.def("bucket_timing", []() { return BucketTimeline::instance().enabled(); });
  m.def("timeline_mark", [](const std::string& name, uint64_t stream) {
    BucketTimeline::instance().mark(name, (cudaStream_t)stream);
  }, py::arg("name"), py::arg("stream"), "Drops a named mark on `stream` into the bucket time line.");
  m.def(
      "timeline_collect",
      []() {
        std::vector<TimelineSpan> spans;
        {
          py::gil_scoped_release rel;
          spans = BucketTimeline::instance().collect();
        }
        py::list out;
        for (auto& sp : spans) {
          py::dict d;
          d["name"] = sp.name;
          d["kind"] = sp.kind;
          d["start_ms"] = sp.start_ms;
          d["end_ms"] = sp.end_ms;
          d["bytes"] = sp.bytes;
          out.append(d);
        }
        return out;
      },
      "Waits for the recorded events and returns [{name, kind: bucket|mark, start_ms, end_ms, bytes}] relative to "
      "the first recorded event; the record is emptied.");
  m.def("set_log_level", [](const std::string& s) { set_log_level(parse_log_level(s.c_str())); });
  m.def("stats", []() {
    auto& s = EngineStats::global();
    py::dict d;
    d["buckets_scheduled"] = s.buckets_scheduled.load();
    d["ops_executed"] = s.ops_executed.load();
    d["fused_launches"] = s.fused_launches.load();
    d["library_fallbacks"] = s.library_fallbacks.load();
    d["staged_copies"] = s.staged_copies.load();
    d["bytes_communicated"] = s.bytes_communicated.load();
    return d;
  });
  m.def("reset_stats", []() {
    auto& s = EngineStats::global();
    s.buckets_scheduled = 0;
    s.ops_executed = 0;
    s.fused_launches = 0;
    s.library_fallbacks = 0;
    s.staged_copies = 0;
    s.bytes_communicated = 0;
  });
  m.def("pool_stats", [](int device) {
    PoolStats s = MemoryPool::for_device(device).stats();
    py::dict d;
    d["device_allocs"] = s.device_allocs;
    d["pulls"] = s.pulls;
    d["bytes_reserved"] = s.bytes_reserved;
    d["bytes_in_use"] = s.bytes_in_use;
    d["guard_violations"] = s.guard_violations;
    return d;
  });
  m.def("pool_set_guard", [](bool on) { MemoryPool::set_guard(on); }, py::arg("on"),
        "Guard regions around pool blocks allocated from now on (also: BAGUA_B200_POOL_GUARD=1).");
  m.def("pool_guard", []() { return MemoryPool::guard(); });
  m.def("pool_check_guards", [](int device) { return MemoryPool::for_device(device).check_guards(); }, py::arg("device"),
        "Number of pool blocks on `device` (-1: host) whose guard regions were overwritten; synchronises the device.");
  m.def("pool_size_class", [](size_t bytes) { return MemoryPool::size_class(bytes); });
  m.def("pool_release_cached", [](int device) { MemoryPool::for_device(device).release_cached(); });
  m.def("shift_one_peer", &shift_one_peer, py::arg("rank"), py::arg("nranks"), py::arg("step"));
  m.def("compressed_buffer_size", [](int n_chunks, int64_t chunk_size, const std::string& dt) {
    DType d = dt == "F16" ? DType::F16 : dt == "BF16" ? DType::BF16 : DType::F32;
    return kernels::compressed_buffer_size(n_chunks, chunk_size, d);
  });

  // telemetry
  m.def("telemetry_init", [](const std::string& addr) { Telemetry::instance().init(addr); });
  m.def("telemetry_enabled", []() { return Telemetry::instance().enabled(); });
  m.def("telemetry_flush", [](int timeout_ms) { return Telemetry::instance().flush(timeout_ms); },
        py::arg("timeout_ms") = 2000, py::call_guard<py::gil_scoped_release>());
  m.def("telemetry_shutdown", []() { Telemetry::instance().shutdown(); }, py::call_guard<py::gil_scoped_release>());
  m.def("telemetry_stats", []() {
    py::dict d;
    d["exported"] = Telemetry::instance().exported();
    d["failed_batches"] = Telemetry::instance().failed_batches();
    return d;
  });

  // raw kernels on torch tensors (tests, optimisers).  `stream` is a cudaStream_t value.
  m.def(
      "k_multi_copy",
      [](std::vector<at::Tensor> tensors, at::Tensor flat, bool gather, uint64_t stream) {
        // tensors packed back to back, in bytes, in list order
        std::vector<kernels::MultiCopySeg> segs;
        unsigned long long off = 0;
        for (auto& t : tensors) {
          BAGUA_CHECK(t.is_contiguous() && t.device() == flat.device(), Tensor,
                      "multi_copy: tensors must be contiguous and on the flat buffer's device");
          if (t.nbytes()) segs.push_back(kernels::MultiCopySeg{t.data_ptr(), off, (unsigned long long)t.nbytes()});
          off += t.nbytes();
        }
        BAGUA_CHECK(flat.is_contiguous() && (unsigned long long)flat.nbytes() >= off, Tensor,
                    "multi_copy: the flat buffer is too small");
        kernels::Ctx c = ctx_of(flat, stream);
        if (!c.is_cuda()) {
          kernels::multi_copy(segs.data(), (int)segs.size(), flat.data_ptr(), (size_t)off, gather, c);
          return;
        }
        at::Tensor table = at::empty({(int64_t)(segs.size() * sizeof(kernels::MultiCopySeg))},
                                     at::TensorOptions().dtype(at::kByte).device(flat.device()));
        BAGUA_CUDA_CHECK(cudaMemcpyAsync(table.data_ptr(), segs.data(), segs.size() * sizeof(kernels::MultiCopySeg),
                                         cudaMemcpyHostToDevice, c.stream));
        kernels::multi_copy((const kernels::MultiCopySeg*)table.data_ptr(), (int)segs.size(), flat.data_ptr(),
                            (size_t)off, gather, c);
        BAGUA_CUDA_CHECK(cudaStreamSynchronize(c.stream));  // `table` and `segs` die with this call
      },
      py::arg("tensors"), py::arg("flat"), py::arg("gather"), py::arg("stream"),
      "Flatten (gather) or unflatten a list of tensors into / out of `flat` (packed back to back) with one kernel.");
  m.def("k_divide_inplace", [](at::Tensor x, float d, uint64_t stream) {
    kernels::divide_inplace(x.data_ptr(), dtype_from_torch(x.scalar_type()), x.numel(), d, ctx_of(x, stream));
  });
  m.def("k_add_inplace", [](at::Tensor x, at::Tensor y, uint64_t stream) {
    check_pair(x, y);
    kernels::add_inplace(x.data_ptr(), y.data_ptr(), dtype_from_torch(x.scalar_type()), x.numel(), ctx_of(x, stream));
  });
  m.def("k_subtract_inplace", [](at::Tensor x, at::Tensor y, uint64_t stream) {
    check_pair(x, y);
    kernels::subtract_inplace(x.data_ptr(), y.data_ptr(), dtype_from_torch(x.scalar_type()), x.numel(),
                              ctx_of(x, stream));
  });
  m.def("k_addmul_inplace", [](at::Tensor x, at::Tensor y, float f, uint64_t stream) {
    check_pair(x, y);
    kernels::addmul_inplace(x.data_ptr(), y.data_ptr(), f, dtype_from_torch(x.scalar_type()), x.numel(),
                            ctx_of(x, stream));
  });
  m.def("k_average_inplace", [](at::Tensor x, at::Tensor y, uint64_t stream) {
    check_pair(x, y);
    kernels::average_inplace(x.data_ptr(), y.data_ptr(), dtype_from_torch(x.scalar_type()), x.numel(),
                             ctx_of(x, stream));
  });
  m.def("k_async_model_average", [](at::Tensor t, at::Tensor reduced, at::Tensor copy, float nranks, uint64_t stream) {
    check_pair(t, reduced);
    check_pair(t, copy);
    BAGUA_CHECK(t.scalar_type() == at::kFloat, Tensor, "async_model_average supports float32 only");
    kernels::async_model_average((float*)t.data_ptr(), (const float*)reduced.data_ptr(), (const float*)copy.data_ptr(),
                                 nranks, t.numel(), ctx_of(t, stream));
  });
  m.def("k_reduce_chunk_inplace", [](at::Tensor x, int n_chunks, int target, bool average, uint64_t stream) {
    BAGUA_CHECK(x.is_contiguous() && n_chunks > 0 && x.numel() % n_chunks == 0, Tensor,
                "tensor must be contiguous and divisible into chunks");
    kernels::reduce_chunk_inplace(x.data_ptr(), dtype_from_torch(x.scalar_type()), x.numel() / n_chunks, n_chunks,
                                  target, average, ctx_of(x, stream));
  });
  m.def(
      "k_sgd_momentum_flat",
      [](at::Tensor p, at::Tensor g, at::Tensor buf, float lr, float momentum, float dampening, float wd, bool nesterov,
         bool first_step, uint64_t stream) {
        check_pair(p, g);
        check_pair(p, buf);
        BAGUA_CHECK(p.scalar_type() == at::kFloat, Tensor, "fused SGD works on float32 flat buffers");
        kernels::sgd_momentum_flat((float*)p.data_ptr(), (const float*)g.data_ptr(), (float*)buf.data_ptr(), p.numel(),
                                   lr, momentum, dampening, wd, nesterov, first_step, ctx_of(p, stream));
      },
      py::arg("param"), py::arg("grad"), py::arg("momentum_buffer"), py::arg("lr"), py::arg("momentum"),
      py::arg("dampening"), py::arg("weight_decay"), py::arg("nesterov"), py::arg("first_step"), py::arg("stream"));

  m.def(
      "k_sgd_momentum_flat_shadow",
      [](at::Tensor p, at::Tensor g, at::Tensor buf, at::Tensor shadow, float lr, float momentum, float dampening,
         float wd, bool nesterov, bool first_step, uint64_t stream) {
        check_pair(p, g);
        check_pair(p, buf);
        BAGUA_CHECK(p.scalar_type() == at::kFloat, Tensor, "fused SGD works on float32 flat buffers");
        BAGUA_CHECK(shadow.scalar_type() == at::kBFloat16 && shadow.is_contiguous() && shadow.numel() == p.numel() &&
                        shadow.device() == p.device(),
                    Tensor, "the shadow must be a contiguous bf16 tensor of the parameters' size on their device");
        kernels::sgd_momentum_flat_shadow((float*)p.data_ptr(), (const float*)g.data_ptr(), (float*)buf.data_ptr(),
                                          shadow.data_ptr(), p.numel(), lr, momentum, dampening, wd, nesterov,
                                          first_step, ctx_of(p, stream));
      },
      py::arg("param"), py::arg("grad"), py::arg("momentum_buffer"), py::arg("bf16_shadow"), py::arg("lr"),
      py::arg("momentum"), py::arg("dampening"), py::arg("weight_decay"), py::arg("nesterov"), py::arg("first_step"),
      py::arg("stream"));

  // ---- fused bias + ReLU for channels-last bf16 activations (model-side kernels) ----
  // An activation is either [rows, C] contiguous or [N, C, H, W] in channels-last memory format.
  auto rows_and_channels = [](const at::Tensor& t, int64_t* rows, int* C) {
    BAGUA_CHECK((t.is_cuda() || t.is_cpu()) && t.scalar_type() == at::kBFloat16, Tensor,
                "fused bias+ReLU works on bf16 tensors (sm_100a kernels on CUDA, plain loops on the host)");
    if (t.dim() == 2 && t.is_contiguous()) {
      *rows = t.size(0);
      *C = (int)t.size(1);
    } else {
      BAGUA_CHECK(t.dim() == 4 && t.is_contiguous(at::MemoryFormat::ChannelsLast), Tensor,
                  "fused bias+ReLU needs a [rows, C] tensor or a channels-last [N, C, H, W] tensor");
      *rows = t.size(0) * t.size(2) * t.size(3);
      *C = (int)t.size(1);
    }
  };
  m.def("k_bias_relu_supported", [](int64_t rows, int C) { return model_ops::bias_relu_supported(rows, C); });
  m.def(
      "k_bias_relu_",
      [rows_and_channels](at::Tensor z, at::Tensor bias, uint64_t stream) {
        int64_t rows;
        int C;
        rows_and_channels(z, &rows, &C);
        BAGUA_CHECK(bias.device() == z.device() && bias.scalar_type() == at::kBFloat16 && bias.is_contiguous() &&
                        bias.numel() == C,
                    Tensor, "bias must be a contiguous bf16 vector with one entry per channel, on the activation's device");
        if (z.is_cuda())
          model_ops::bias_relu_inplace_bf16(z.data_ptr(), bias.data_ptr(), rows, C, (cudaStream_t)stream);
        else
          model_ops::bias_relu_inplace_bf16_host(z.data_ptr(), bias.data_ptr(), rows, C);
      },
      py::arg("activation"), py::arg("bias"), py::arg("stream"), "activation = max(activation + bias, 0), in place.");
  m.def(
      "k_bias_relu_backward",
      [rows_and_channels](at::Tensor dy, at::Tensor y, at::Tensor dz, at::Tensor db, uint64_t stream) {
        int64_t rows, r2, r3;
        int C, C2, C3;
        rows_and_channels(dy, &rows, &C);
        rows_and_channels(y, &r2, &C2);
        rows_and_channels(dz, &r3, &C3);
        BAGUA_CHECK(rows == r2 && rows == r3 && C == C2 && C == C3, Tensor, "dy, y and dz must have the same shape");
        BAGUA_CHECK(db.device() == dy.device() && y.device() == dy.device() && dz.device() == dy.device() &&
                        db.scalar_type() == at::kFloat && db.is_contiguous() && db.numel() == C,
                    Tensor, "db must be a contiguous fp32 vector with one entry per channel; all tensors on one device");
        if (!dy.is_cuda()) {
          model_ops::bias_relu_backward_bf16_host(dy.data_ptr(), y.data_ptr(), dz.data_ptr(), (float*)db.data_ptr(), rows, C);
          return;
        }
        const size_t need = model_ops::bias_relu_backward_scratch_bytes(rows, C);
        BAGUA_CHECK(need > 0, Tensor, "fused bias+ReLU backward: unsupported shape");
        auto scratch = PoolRawTensor::allocate((int)dy.device().index(), DType::U8, (int64_t)need, stream);
        model_ops::bias_relu_backward_bf16(dy.data_ptr(), y.data_ptr(), dz.data_ptr(), (float*)db.data_ptr(), rows, C,
                                           scratch->data_ptr(), (cudaStream_t)stream);
      },
      py::arg("grad_output"), py::arg("output"), py::arg("grad_pre_activation"), py::arg("grad_bias"), py::arg("stream"),
      "grad_pre_activation = grad_output * [output > 0]; grad_bias[c] = column sums of it (fp32).");

  // 2x2 / stride-2 max pooling on channels-last bf16 [N, C, H, W] tensors
  auto nhwc_dims = [](const at::Tensor& t, int64_t* N, int64_t* H, int64_t* W, int* C) {
    BAGUA_CHECK((t.is_cuda() || t.is_cpu()) && t.scalar_type() == at::kBFloat16 && t.dim() == 4 &&
                    t.is_contiguous(at::MemoryFormat::ChannelsLast),
                Tensor, "fused max-pool works on channels-last bf16 [N, C, H, W] tensors");
    *N = t.size(0);
    *C = (int)t.size(1);
    *H = t.size(2);
    *W = t.size(3);
  };
  m.def("k_maxpool2x2_supported",
        [](int64_t N, int64_t H, int64_t W, int C) { return model_ops::maxpool2x2_supported(N, H, W, C); });
  m.def(
      "k_maxpool2x2_forward",
      [nhwc_dims](at::Tensor x, at::Tensor y, uint64_t stream) {
        int64_t N, H, W, N2, H2, W2;
        int C, C2;
        nhwc_dims(x, &N, &H, &W, &C);
        nhwc_dims(y, &N2, &H2, &W2, &C2);
        BAGUA_CHECK(N2 == N && C2 == C && H2 * 2 == H && W2 * 2 == W, Tensor, "y must be [N, C, H/2, W/2]");
        BAGUA_CHECK(x.device() == y.device(), Tensor, "input and output must be on one device");
        if (x.is_cuda())
          model_ops::maxpool2x2_forward_bf16(x.data_ptr(), y.data_ptr(), N, H, W, C, (cudaStream_t)stream);
        else
          model_ops::maxpool2x2_forward_bf16_host(x.data_ptr(), y.data_ptr(), N, H, W, C);
      },
      py::arg("input"), py::arg("output"), py::arg("stream"));
  m.def(
      "k_maxpool2x2_backward",
      [nhwc_dims](at::Tensor x, at::Tensor dy, at::Tensor dx, uint64_t stream) {
        int64_t N, H, W, N2, H2, W2, N3, H3, W3;
        int C, C2, C3;
        nhwc_dims(x, &N, &H, &W, &C);
        nhwc_dims(dy, &N2, &H2, &W2, &C2);
        nhwc_dims(dx, &N3, &H3, &W3, &C3);
        BAGUA_CHECK(N2 == N && C2 == C && H2 * 2 == H && W2 * 2 == W && N3 == N && C3 == C && H3 == H && W3 == W, Tensor,
                    "dy must be [N, C, H/2, W/2] and dx [N, C, H, W]");
        BAGUA_CHECK(x.device() == dy.device() && x.device() == dx.device(), Tensor, "all tensors must be on one device");
        if (x.is_cuda())
          model_ops::maxpool2x2_backward_bf16(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), N, H, W, C, (cudaStream_t)stream);
        else
          model_ops::maxpool2x2_backward_bf16_host(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), N, H, W, C);
      },
      py::arg("input"), py::arg("grad_output"), py::arg("grad_input"), py::arg("stream"));

  // bias + ReLU followed by 2x2 pooling in one pass each way
  m.def(
      "k_bias_relu_pool_",
      [nhwc_dims](at::Tensor y, at::Tensor p, at::Tensor bias, uint64_t stream) {
        int64_t N, H, W, N2, H2, W2;
        int C, C2;
        nhwc_dims(y, &N, &H, &W, &C);
        nhwc_dims(p, &N2, &H2, &W2, &C2);
        BAGUA_CHECK(N2 == N && C2 == C && H2 * 2 == H && W2 * 2 == W && p.device() == y.device(), Tensor,
                    "the pooled output must be [N, C, H/2, W/2] on the activation's device");
        BAGUA_CHECK(bias.device() == y.device() && bias.scalar_type() == at::kBFloat16 && bias.is_contiguous() &&
                        bias.numel() == C,
                    Tensor, "bias must be a contiguous bf16 vector with one entry per channel, on the activation's device");
        if (y.is_cuda())
          model_ops::bias_relu_pool_bf16(y.data_ptr(), p.data_ptr(), bias.data_ptr(), N, H, W, C, (cudaStream_t)stream);
        else
          model_ops::bias_relu_pool_bf16_host(y.data_ptr(), p.data_ptr(), bias.data_ptr(), N, H, W, C);
      },
      py::arg("activation"), py::arg("pooled"), py::arg("bias"), py::arg("stream"),
      "activation = max(activation + bias, 0) in place; pooled = its 2x2 / stride-2 maximum.");
  m.def(
      "k_bias_relu_pool_backward",
      [nhwc_dims](at::Tensor dp, at::Tensor y, at::Tensor dz, at::Tensor db, uint64_t stream) {
        int64_t N, H, W, N2, H2, W2, N3, H3, W3;
        int C, C2, C3;
        nhwc_dims(y, &N, &H, &W, &C);
        nhwc_dims(dp, &N2, &H2, &W2, &C2);
        nhwc_dims(dz, &N3, &H3, &W3, &C3);
        BAGUA_CHECK(N2 == N && C2 == C && H2 * 2 == H && W2 * 2 == W && N3 == N && C3 == C && H3 == H && W3 == W, Tensor,
                    "grad_pooled must be [N, C, H/2, W/2] and grad_pre_activation [N, C, H, W]");
        BAGUA_CHECK(dp.device() == y.device() && dz.device() == y.device() && db.device() == y.device() &&
                        db.scalar_type() == at::kFloat && db.is_contiguous() && db.numel() == C,
                    Tensor, "db must be a contiguous fp32 vector with one entry per channel; all tensors on one device");
        if (!y.is_cuda()) {
          model_ops::bias_relu_pool_backward_bf16_host(dp.data_ptr(), y.data_ptr(), dz.data_ptr(), (float*)db.data_ptr(), N, H,
                                                       W, C);
          return;
        }
        const size_t need = model_ops::bias_relu_backward_scratch_bytes(N * (H / 2) * (W / 2), C);
        BAGUA_CHECK(need > 0, Tensor, "fused bias+ReLU+pool backward: unsupported shape");
        auto scratch = PoolRawTensor::allocate((int)y.device().index(), DType::U8, (int64_t)need, stream);
        model_ops::bias_relu_pool_backward_bf16(dp.data_ptr(), y.data_ptr(), dz.data_ptr(), (float*)db.data_ptr(), N, H, W, C,
                                                scratch->data_ptr(), (cudaStream_t)stream);
      },
      py::arg("grad_pooled"), py::arg("output"), py::arg("grad_pre_activation"), py::arg("grad_bias"), py::arg("stream"),
      "Backward of k_bias_relu_pool_: routes grad_pooled to each window's first maximum where it is positive.");

  // ---- single-GPU emulation of the fused kernels (all ranks in one cooperative launch) ----
  py::class_<fused::EmulatedArena>(m, "EmulatedArena")
      .def(py::init<int, int, size_t>(), py::arg("nranks"), py::arg("device"), py::arg("staging_bytes"))
      .def("nranks", &fused::EmulatedArena::nranks)
      .def("epoch", &fused::EmulatedArena::epoch)
      .def("set_deadline_ms", &fused::EmulatedArena::set_deadline_ms)
      .def(
          "allreduce",
          [](fused::EmulatedArena& a, std::vector<at::Tensor> in, std::vector<at::Tensor> out, bool average,
             const std::string& mode, int blocks) {
            BAGUA_CHECK(!in.empty() && in.size() == out.size(), Tensor, "one input and one output per rank");
            std::vector<const void*> pi;
            std::vector<void*> po;
            for (size_t r = 0; r < in.size(); ++r) {
              check_pair(in[r], out[r]);
              check_pair(in[0], in[r]);
              pi.push_back(in[r].data_ptr());
              po.push_back(out[r].data_ptr());
            }
            const auto md = mode == "oneshot"         ? fused::EmuAllreduceMode::OneShot
                            : mode == "twoshot"       ? fused::EmuAllreduceMode::TwoShot
                            : mode == "symmetric_tma" ? fused::EmuAllreduceMode::SymmetricTma
                                                      : fused::EmuAllreduceMode::Symmetric;
            py::gil_scoped_release rel;
            a.allreduce(pi, po, in[0].numel(), dtype_from_torch(in[0].scalar_type()),
                        average ? 1.0f / (float)a.nranks() : 1.0f, md, blocks);
          },
          py::arg("inputs"), py::arg("outputs"), py::arg("average"), py::arg("mode"), py::arg("blocks"))
      .def(
          "pair_average",
          [](fused::EmulatedArena& a, std::vector<at::Tensor> in, std::vector<at::Tensor> out, std::vector<int> peers,
             int blocks, bool symmetric) {
            std::vector<const void*> pi;
            std::vector<void*> po;
            for (size_t r = 0; r < in.size(); ++r) {
              check_pair(in[r], out[r]);
              pi.push_back(in[r].data_ptr());
              po.push_back(out[r].data_ptr());
            }
            py::gil_scoped_release rel;
            a.pair_average(pi, po, in[0].numel(), dtype_from_torch(in[0].scalar_type()), peers, blocks, symmetric);
          },
          py::arg("inputs"), py::arg("outputs"), py::arg("peers"), py::arg("blocks"), py::arg("symmetric") = false)
      .def(
          "bytegrad",
          [](fused::EmulatedArena& a, std::vector<at::Tensor> buckets, bool average, int blocks) {
            std::vector<void*> p;
            for (auto& t : buckets) {
              check_pair(buckets[0], t);
              p.push_back(t.data_ptr());
            }
            py::gil_scoped_release rel;
            a.bytegrad(p, buckets[0].numel(), dtype_from_torch(buckets[0].scalar_type()), average, blocks);
          },
          py::arg("buckets"), py::arg("average"), py::arg("blocks"))
      .def(
          "lp_ring",
          [](fused::EmulatedArena& a, std::vector<at::Tensor> x, std::vector<at::Tensor> w, std::vector<at::Tensor> l,
             std::vector<at::Tensor> r, int blocks) {
            std::vector<void*> px, pw, pl, pr;
            for (size_t k = 0; k < x.size(); ++k) {
              check_pair(x[0], x[k]);
              check_pair(x[k], w[k]);
              check_pair(x[k], l[k]);
              check_pair(x[k], r[k]);
              px.push_back(x[k].data_ptr());
              pw.push_back(w[k].data_ptr());
              pl.push_back(l[k].data_ptr());
              pr.push_back(r[k].data_ptr());
            }
            py::gil_scoped_release rel;
            a.lp_ring(px, pw, pl, pr, x[0].numel(), dtype_from_torch(x[0].scalar_type()), blocks);
          },
          py::arg("x"), py::arg("weight"), py::arg("left"), py::arg("right"), py::arg("blocks"))
      .def(
          "alltoall_v",
          [](fused::EmulatedArena& a, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
             std::vector<int64_t> bytes) {
            std::vector<const void*> pi;
            std::vector<void*> po;
            const size_t n = (size_t)a.nranks();
            BAGUA_CHECK(in.size() == n && out.size() == n && bytes.size() == n * n, Tensor,
                        "one input and one output per rank and an N x N table of byte counts expected");
            for (size_t r = 0; r < n; ++r) {
              BAGUA_CHECK(in[r].is_cuda() && in[r].is_contiguous() && out[r].is_cuda() && out[r].is_contiguous(), Tensor,
                          "buffers must be contiguous CUDA tensors");
              int64_t sent = 0, received = 0;
              for (size_t q = 0; q < n; ++q) {
                sent += bytes[r * n + q];
                received += bytes[q * n + r];
              }
              BAGUA_CHECK((size_t)sent <= in[r].nbytes() && (size_t)received <= out[r].nbytes(), Tensor,
                          "the size table does not fit the buffers of rank " << r);
              pi.push_back(in[r].data_ptr());
              po.push_back(out[r].data_ptr());
            }
            py::gil_scoped_release rel;
            a.alltoall_v(pi, po, bytes, 4);
          },
          py::arg("inputs"), py::arg("outputs"), py::arg("bytes"),
          "All-to-all with per-pair sizes: rank s sends bytes[s * N + d] bytes to rank d, segments packed back "
          "to back on both sides.")
      .def(
          "collective",
          [](fused::EmulatedArena& a, const std::string& kind, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
             bool symmetric, int root, bool average, int blocks) {
            fused::EmuCollective k;
            if (kind == "allgather") k = fused::EmuCollective::AllGather;
            else if (kind == "alltoall") k = fused::EmuCollective::AllToAll;
            else if (kind == "reduce_scatter") k = fused::EmuCollective::ReduceScatter;
            else if (kind == "broadcast_direct") k = fused::EmuCollective::BroadcastDirect;
            else if (kind == "broadcast_twophase") k = fused::EmuCollective::BroadcastTwoPhase;
            else if (kind == "barrier") k = fused::EmuCollective::Barrier;
            else if (kind == "scatter") k = fused::EmuCollective::Scatter;
            else if (kind == "gather") k = fused::EmuCollective::Gather;
            else if (kind == "reduce_direct") k = fused::EmuCollective::ReduceDirect;
            else if (kind == "reduce_twophase") k = fused::EmuCollective::ReduceTwoPhase;
            else throw BaguaError(ErrorKind::Communicator, "unknown collective '" + kind + "'");
            std::vector<const void*> pi;
            std::vector<void*> po;
            size_t chunk_bytes = 0;
            DType dt = DType::F32;
            if (k != fused::EmuCollective::Barrier) {
              BAGUA_CHECK(!out.empty(), Tensor, "one output per rank expected");
              for (auto& t : out) {
                check_pair(out[0], t);
                po.push_back(t.data_ptr());
              }
              for (auto& t : in) {
                BAGUA_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == out[0].scalar_type(), Tensor,
                            "inputs must be contiguous CUDA tensors of the outputs' dtype");
                pi.push_back(t.data_ptr());
              }
              dt = dtype_from_torch(out[0].scalar_type());
              const size_t n = (size_t)a.nranks();
              if (k == fused::EmuCollective::AllGather) chunk_bytes = out[0].nbytes() / n;
              else if (k == fused::EmuCollective::AllToAll) chunk_bytes = out[0].nbytes() / n;
              else if (k == fused::EmuCollective::Gather) chunk_bytes = out[0].nbytes() / n;
              else chunk_bytes = out[0].nbytes();  // reduce-scatter / scatter output, broadcast / reduce buffer
              if (k == fused::EmuCollective::AllGather || k == fused::EmuCollective::AllToAll)
                BAGUA_CHECK(out[0].nbytes() % n == 0, Tensor, "output size must be divisible by the number of ranks");
            }
            py::gil_scoped_release rel;
            a.collective(k, pi, po, chunk_bytes, dt, average ? 1.0f / (float)a.nranks() : 1.0f, root, symmetric, blocks);
          },
          py::arg("kind"), py::arg("inputs"), py::arg("outputs"), py::arg("symmetric") = false, py::arg("root") = 0,
          py::arg("average") = false, py::arg("blocks") = 4,
          "Runs one of the communicator collectives (allgather, alltoall, reduce_scatter, broadcast_direct, "
          "broadcast_twophase, scatter, gather, reduce_direct, reduce_twophase, barrier) for all virtual ranks in "
          "one cooperative launch.");

  m.def("release_multicast_slabs", []() { return release_all_multicast_slabs(); },
        "Drops every NVSwitch multicast binding this process holds (called at interpreter exit).");
  m.def(
      "debug_wait_timeout",
      [](int device, double wait_ms) {
        DeviceStatus s;
        {
          py::gil_scoped_release rel;
          s = fused::debug_wait_timeout(device, wait_ms);
        }
        py::dict d;
        d["code"] = s.code;
        d["phase"] = s.phase;
        d["peer"] = s.peer;
        d["block"] = s.block;
        d["epoch"] = s.epoch;
        d["seen"] = s.seen;
        return d;
      },
      py::arg("device"), py::arg("wait_ms"),
      "Runs a kernel whose only wait can never be satisfied and returns the status record it left.");
}
