"""`with_bagua`: wrap a model so that an algorithm's communication overlaps its backward pass.

The wrapper is the trainer-side half of the engine's contract
(reference: bagua-core-internal/src/lib.rs:270-337 and the call sequence in
bagua-core-py/src/lib.rs:316-349):

1. parameters are broadcast from rank 0;
2. the algorithm names the tensors to communicate (gradients or weights), they are packed
   into flat buckets in reverse registration order (the order gradients become ready) and
   registered with `register_ordered_buckets`;
3. a post-accumulate-grad hook per parameter calls `mark_communication_ready`; only the
   last tensor of each bucket records a CUDA event (earlier ones are covered by it, being on
   the same stream), so a bucket costs one event, not one per tensor;
4. after backward `wait_pending_comm_ops()` returns once the worker has queued every
   bucket's kernel, and the compute stream is made to wait on the communication stream.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .._native import C as _C
from .bucket import ALIGN_ELEMS_PER_RANK, BaguaBucket, BaguaTensor
from .communication import BaguaProcessGroup, get_process_group


class BaguaModule(nn.Module):
    """A model prepared by :func:`with_bagua`.  Call it like the original module; call
    ``optimizer.step()`` as usual — gradient synchronisation has finished (stream-wise) when
    ``backward()`` returns."""

    def __init__(self, module: nn.Module, optimizers: Sequence[torch.optim.Optimizer], algorithm,
                 process_group: Optional[BaguaProcessGroup] = None, bucket_bytes: int = 10 * 1024 ** 2,
                 broadcast_parameters: bool = True):
        super().__init__()
        self.module = module
        self.bagua_optimizers = list(optimizers)
        self.bagua_algorithm = algorithm
        self.pg = process_group or get_process_group()
        self.bucket_bytes = bucket_bytes
        self.bagua_buckets: List[BaguaBucket] = []
        self.bagua_train_step_counter = 0
        self._hooks = []
        self._events = {}
        self._pending_backward = False
        self._in_no_sync = False
        self._named_params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        if broadcast_parameters and self.pg.world_size > 1:
            self._broadcast_parameters()
        self._reset()

    # ---- setup -----------------------------------------------------------------------
    def _broadcast_parameters(self):
        with torch.no_grad():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                dist.broadcast(t.data, src=0)

    def _reset(self):
        """(Re)build tensors, buckets, ops and hooks; called again when the algorithm asks for it."""
        self.pg.backend.wait_pending_comm_ops()
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        algo = self.bagua_algorithm
        # flat buffers of the buckets being replaced: a bucket whose tensors already sit in one of them,
        # in the same order, keeps it (symmetric memory is never given back to the arena, so a rebuild
        # with an unchanged layout must not take a second set)
        self._prev_flats = [b.flattened for b in self.bagua_buckets if b.flattened is not None]
        tensors = algo.init_tensors(self)
        groups = algo.tensors_to_buckets(self, tensors)
        align = ALIGN_ELEMS_PER_RANK * max(1, self.pg.world_size)
        self.bagua_buckets = [
            BaguaBucket(g, f"bucket_{i}", flatten=algo.flatten_buckets, alignment=align, allocator=self._alloc_flat)
            for i, g in enumerate(groups)
        ]
        self._prev_flats = []
        for b in self.bagua_buckets:
            algo.init_operations(self, b)
        for opt in self.bagua_optimizers:
            if hasattr(opt, "bagua_attach"):
                opt.bagua_attach(self)
        self.pg.backend.register_ordered_buckets([b.backend_bucket for b in self.bagua_buckets])
        # per-bucket bookkeeping for the one-event-per-bucket rule
        # (the hooks run once per parameter per step on the thread that launches the backward kernels:
        # they reach their bucket and its countdown through attributes, not through look-ups by name)
        for b in self.bagua_buckets:
            b._pending = len(b.tensors)
            for t in b.tensors:
                t._bucket = b
                t._step = -1
        self._mark_ready_native = self.pg.backend.mark_communication_ready
        self._on_cuda = bool(self.pg.is_cuda)
        self._hooks.extend(algo.init_backward_hooks(self))
        self._hooks.extend(algo.init_forward_pre_hooks(self))
        self._post_backward = algo.init_post_backward_hook(self)
        self._post_step = algo.init_post_optimizer_step_hook(self)
        self._wrap_optimizer_steps()
        self._arm()

    def _alloc_flat(self, numel, dtype, device, tensors=()):
        """Bucket storage: symmetric memory of the global communicator when there are peers
        (the engine then all-reduces the bucket in place over NVLink with no staging copy);
        None → the bucket falls back to an ordinary zero tensor.  Collective: every rank
        builds the same buckets in the same order."""
        import os

        for old in getattr(self, "_prev_flats", ()):
            if old.numel() == numel and old.dtype == dtype and old.device == device and tensors:
                off, es, base = 0, old.element_size(), old.data_ptr()
                for t in tensors:
                    if t.tensor.dtype != dtype or t.tensor.data_ptr() != base + off * es:
                        break
                    off += t.tensor.numel()
                else:
                    return old

        if (not self.pg.is_cuda or self.pg.world_size < 2 or os.environ.get("BAGUA_B200_SYMMETRIC", "1") == "0"
                or os.environ.get("BAGUA_B200_FUSED", "1") == "0"):
            return None
        if dtype not in (torch.float32, torch.float16, torch.bfloat16):
            return None
        return self._bucket_comm().alloc_symmetric(int(numel), dtype)

    def _bucket_comm(self):
        """The communicator whose fused kernels will reduce the buckets: symmetric memory must come from
        its arena.  A hierarchical algorithm on one node reduces over the intra-node communicator."""
        if getattr(self.bagua_algorithm, "hierarchical", False):
            self.pg.ensure_hierarchical()
            intra = self.pg.intra_comm
            if intra is not None and intra.nranks() == self.pg.world_size:
                return intra
        return self.pg.global_comm

    def _arm(self):
        for b in self.bagua_buckets:
            b._pending = len(b.tensors)

    def _wrap_optimizer_steps(self):
        for opt in self.bagua_optimizers:
            if getattr(opt, "_bagua_wrapped", None) is self:
                continue
            inner_step = opt.step if not hasattr(opt, "_bagua_inner_step") else opt._bagua_inner_step

            def step(*a, _inner=inner_step, **kw):
                out = _inner(*a, **kw)
                self._post_step()
                return out

            opt._bagua_inner_step = inner_step
            opt.step = step
            opt._bagua_wrapped = self

    # ---- the hot path ------------------------------------------------------------------
    def mark_ready(self, t: BaguaTensor):
        """Tell the engine `t` holds its final value for this step (called from hooks)."""
        b = t._bucket
        b._pending -= 1
        t._step = self.bagua_train_step_counter
        ev_ptr = 0
        if b._pending == 0 and self._on_cuda:
            ev = self._events.get(b.name)
            if ev is None:
                ev = self._events[b.name] = torch.cuda.Event(enable_timing=False, blocking=False)
            ev.record()
            ev_ptr = ev.cuda_event
        self._mark_ready_native(t.backend_tensor, ev_ptr)

    def _timeline_mark(self, name):
        """A named point on the compute stream in the engine's device time line (when it is recording)."""
        if self._on_cuda and _C.bucket_timing():
            _C.timeline_mark(name, torch.cuda.current_stream().cuda_stream)

    def flush_unready(self):
        """Marks every tensor that no hook has marked in this step, so that its bucket is still
        communicated: a parameter that took no part in this step's loss gets no gradient hook, and
        its bucket would otherwise wait for it forever (and hold back every bucket behind it).
        Its gradient goes into the reduction as it is (zero after `zero_grad`)."""
        step = self.bagua_train_step_counter
        for b in self.bagua_buckets:
            if b._pending > 0:
                for t in b.tensors:
                    if t._step != step:
                        self.mark_ready(t)

    def forward(self, *args, **kwargs):
        self._timeline_mark("step_begin")
        out = self.module(*args, **kwargs)
        if torch.is_grad_enabled() and not self._in_no_sync:
            self._pending_backward = True
            # run the post-backward hook when the autograd engine finishes this graph
            if not getattr(self, "_callback_queued", False):
                self._queue_post_backward(out)
        return out

    def _queue_post_backward(self, out):
        tensors = [t for t in _flatten_outputs(out) if isinstance(t, torch.Tensor) and t.requires_grad]
        if not tensors:
            return
        outer = self

        def on_grad(_g):
            if not getattr(outer, "_callback_queued", False):
                outer._callback_queued = True
                torch.autograd.Variable._execution_engine.queue_callback(outer._after_backward)
            return None

        # every output: the loss may depend on any of them (an auxiliary output listed first need not
        # take part in it); the flag makes the callback run once per backward pass whichever fire
        for t in tensors:
            t.register_hook(on_grad)

    def _after_backward(self):
        self._callback_queued = False
        if not self._pending_backward:
            return
        self._pending_backward = False
        self._timeline_mark("backward_end")
        self._post_backward()
        self._arm()
        self.bagua_train_step_counter += 1
        if self.bagua_algorithm.need_reset(self):
            self._reset()

    def no_sync(self):
        """Context manager: accumulate gradients locally without communicating."""
        outer = self

        class _Ctx:
            def __enter__(self_inner):
                outer._in_no_sync = True

            def __exit__(self_inner, *exc):
                outer._in_no_sync = False

        return _Ctx()

    # ---- checkpointing ---------------------------------------------------------------
    def bagua_state_dict(self):
        """State of the communication ops that is not in the model/optimizer state dicts."""
        return {
            "step": self.bagua_train_step_counter,
            "ops": [b.backend_bucket.ops_state() for b in self.bagua_buckets],
            "algorithm": self.bagua_algorithm.state_dict(self),
        }

    def load_bagua_state_dict(self, state):
        self.bagua_train_step_counter = state["step"]
        for b, st in zip(self.bagua_buckets, state["ops"]):
            b.backend_bucket.load_ops_state([[tuple(kv) for kv in op] for op in st])
        self.bagua_algorithm.load_state_dict(self, state.get("algorithm", {}))


def _flatten_outputs(out):
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, (list, tuple)):
        r = []
        for o in out:
            r.extend(_flatten_outputs(o))
        return r
    if isinstance(out, dict):
        r = []
        for o in out.values():
            r.extend(_flatten_outputs(o))
        return r
    return []


def with_bagua(module: nn.Module, optimizers: Sequence[torch.optim.Optimizer], algorithm,
               process_group: Optional[BaguaProcessGroup] = None, bucket_bytes: int = 10 * 1024 ** 2,
               broadcast_parameters: bool = True) -> BaguaModule:
    """Prepare `module` for distributed training with `algorithm` (see
    `bagua_core_b200.parallel.algorithms`)."""
    return BaguaModule(module, optimizers, algorithm, process_group, bucket_bytes, broadcast_parameters)
