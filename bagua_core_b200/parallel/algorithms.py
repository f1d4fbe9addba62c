"""Training algorithms built on the engine's communication ops.

Each algorithm says which tensors are communicated (gradients or weights), how they are
bucketed, which engine op every bucket runs, and where in the training step the tensors
are marked ready.  They correspond to the six ops of the reference
(bagua-core-internal/src/comm_ops/*.rs) the way the external trainer drives them:

* GradientAllReduceAlgorithm         → centralized full precision (O1)
* ByteGradAlgorithm                  → centralized low precision, MinMaxUInt8 (O2)
* DecentralizedAlgorithm             → decentralized full precision, all / shift_one (O3)
* LowPrecisionDecentralizedAlgorithm → decentralized low precision ring (O4)
* QAdamAlgorithm                     → O1 during warm-up, then O2 on momentum buckets
* AsyncModelAverageAlgorithm         → decentralized asynchronous (O5), timer-driven
"""
from __future__ import annotations

import threading
from typing import List

import torch

from .bucket import BaguaBucket, BaguaTensor, split_into_buckets


class Algorithm:
    """Base class; the defaults communicate gradients during backward."""

    flatten_buckets = True

    def need_reset(self, bm) -> bool:
        return False

    # -- what is communicated ---------------------------------------------------------
    def init_tensors(self, bm) -> List[BaguaTensor]:
        """Gradients, in reverse registration order (≈ the order they become ready)."""
        tensors = []
        for name, p in reversed(bm._named_params):
            if p.grad is None:
                p.grad = torch.zeros_like(p, memory_format=torch.preserve_format)
            tensors.append(BaguaTensor(p.grad, name + ".grad", owner=p, kind="grad"))
        return tensors

    def tensors_to_buckets(self, bm, tensors):
        return split_into_buckets(tensors, bm.bucket_bytes)

    def init_operations(self, bm, bucket: BaguaBucket):
        raise NotImplementedError

    # -- when ---------------------------------------------------------------------------
    def init_backward_hooks(self, bm):
        hooks = []
        by_param = {id(t.owner): t for b in bm.bagua_buckets for t in b.tensors if t.owner is not None}

        def make(t):
            def hook(param):
                if bm._in_no_sync:
                    return
                if param.grad is not t.tensor:
                    # someone replaced .grad (e.g. zero_grad(set_to_none=True)): move the new
                    # gradient into the bucket and make the bucket view the .grad again
                    with torch.no_grad():
                        t.tensor.copy_(param.grad)
                    param.grad = t.tensor
                bm.mark_ready(t)

            return hook

        for _, p in bm._named_params:
            t = by_param.get(id(p))
            if t is not None:
                hooks.append(p.register_post_accumulate_grad_hook(make(t)))
        return hooks

    def init_forward_pre_hooks(self, bm):
        return []

    def init_post_backward_hook(self, bm):
        def hook():
            self.flush_unready(bm)
            bm.pg.backend.wait_pending_comm_ops()
            bm.pg.wait_comm_stream()

        return hook

    def flush_unready(self, bm):
        """Gradients that did not arrive in this backward pass (parameters the loss did not use)."""
        bm.flush_unready()

    def init_post_optimizer_step_hook(self, bm):
        return lambda: None

    def state_dict(self, bm):
        return {}

    def load_state_dict(self, bm, state):
        pass


class GradientAllReduceAlgorithm(Algorithm):
    """Synchronous data parallelism: average (or sum) gradients across all ranks."""

    def __init__(self, hierarchical: bool = False, average: bool = True, scattergather: bool = False):
        self.hierarchical = hierarchical
        self.average = average
        self.scattergather = scattergather

    def init_operations(self, bm, bucket):
        bucket.clear_ops()
        bucket.append_centralized_synchronous_op(bm.pg, hierarchical=self.hierarchical, average=self.average,
                                                 scattergather=self.scattergather)


class ByteGradAlgorithm(Algorithm):
    """Gradients are quantised to 8 bits (per-chunk min/max) for both the scatter-reduce and
    the all-gather half of the all-reduce."""

    def __init__(self, hierarchical: bool = False, average: bool = True):
        self.hierarchical = hierarchical
        self.average = average

    def init_operations(self, bm, bucket):
        bucket.clear_ops()
        bucket.append_centralized_synchronous_op(bm.pg, hierarchical=self.hierarchical, average=self.average,
                                                 scattergather=True, compression="MinMaxUInt8")


class _WeightAlgorithm(Algorithm):
    """Shared by the algorithms that communicate weights instead of gradients."""

    def init_tensors(self, bm):
        return [BaguaTensor(p, name, owner=p, kind="weight") for name, p in bm._named_params]

    def init_backward_hooks(self, bm):
        return []

    def _mark_all(self, bm):
        for b in bm.bagua_buckets:
            for t in b.tensors:
                bm.mark_ready(t)
        bm._arm()


class DecentralizedAlgorithm(_WeightAlgorithm):
    """Decentralized SGD: every `communication_interval` steps each rank averages its weights
    with all ranks (`all`) or with one rotating partner (`shift_one`).  The exchange starts
    before the forward pass and overlaps forward+backward; the averaged weights replace the
    local ones after backward, before the optimizer applies this step's gradients."""

    def __init__(self, hierarchical: bool = False, peer_selection_mode: str = "all", communication_interval: int = 1):
        assert peer_selection_mode in ("all", "shift_one")
        self.hierarchical = hierarchical
        self.peer_selection_mode = peer_selection_mode
        self.communication_interval = communication_interval

    def init_operations(self, bm, bucket):
        bucket.clear_ops()
        bucket.peer_weight = torch.zeros_like(bucket.flattened)
        bucket.append_decentralized_synchronous_op(bm.pg, bucket.peer_weight, hierarchical=self.hierarchical,
                                                   peer_selection_mode=self.peer_selection_mode)

    def _communicating(self, bm):
        return bm.bagua_train_step_counter % self.communication_interval == 0

    def init_forward_pre_hooks(self, bm):
        def pre(_module, _inputs):
            if torch.is_grad_enabled() and not bm._in_no_sync and self._communicating(bm):
                self._mark_all(bm)

        return [bm.module.register_forward_pre_hook(pre)]

    def init_post_backward_hook(self, bm):
        def hook():
            if not self._communicating(bm):
                return
            bm.pg.backend.wait_pending_comm_ops()
            bm.pg.wait_comm_stream()
            with torch.no_grad():
                for b in bm.bagua_buckets:
                    b.flattened.copy_(b.peer_weight)

        return hook


class LowPrecisionDecentralizedAlgorithm(_WeightAlgorithm):
    """Decentralized SGD on a ring where neighbours exchange 8-bit quantised weight
    differences; every rank keeps replicas of its own and its two neighbours' weights."""

    def __init__(self, hierarchical: bool = False, communication_interval: int = 1):
        self.hierarchical = hierarchical
        self.communication_interval = communication_interval

    def init_operations(self, bm, bucket):
        bucket.clear_ops()
        bucket.weight = bucket.flattened.clone()
        bucket.left_peer_weight = bucket.flattened.clone()
        bucket.right_peer_weight = bucket.flattened.clone()
        bucket.append_low_precision_decentralized_synchronous_op(
            bm.pg, bucket.weight, bucket.left_peer_weight, bucket.right_peer_weight, hierarchical=self.hierarchical)

    def init_post_backward_hook(self, bm):
        return lambda: None

    def init_post_optimizer_step_hook(self, bm):
        def hook():
            # step counter was already advanced by the post-backward callback
            if (bm.bagua_train_step_counter - 1) % self.communication_interval != 0:
                return
            self._mark_all(bm)
            bm.pg.backend.wait_pending_comm_ops()
            bm.pg.wait_comm_stream()

        return hook


class QAdamOptimizer(torch.optim.Optimizer):
    """Adam whose second moment is frozen after `warmup_steps`; from then on the first
    moment is what ranks exchange (8-bit compressed), so the optimizer only applies
    `p -= lr * m / (sqrt(v) + eps)`."""

    def __init__(self, params, lr=1e-3, warmup_steps=100, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.warmup_steps = warmup_steps
        self.step_id = 0
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)

    @torch.no_grad()
    def step(self, closure=None):
        """One multi-tensor call per operation and parameter group instead of one small kernel per
        operation and parameter (for BERT-large: 9 launches instead of about 1500 after warm-up);
        the arithmetic per element is the same sequence of operations."""
        loss = closure() if closure is not None else None
        self.step_id += 1
        warm = self.step_id <= self.warmup_steps
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            # during warm-up a parameter without a gradient is left alone; afterwards `m` was updated
            # (and averaged across ranks) by the algorithm, so every parameter moves
            ps = [p for p in group["params"] if not warm or p.grad is not None]
            if not ps:
                continue
            ms = [self.state[p]["exp_avg"] for p in ps]
            vs = [self.state[p]["exp_avg_sq"] for p in ps]
            if warm:
                gs = [p.grad for p in ps]
                if wd != 0:
                    gs = torch._foreach_add(gs, ps, alpha=wd)
                torch._foreach_mul_(ms, b1)
                torch._foreach_add_(ms, gs, alpha=1 - b1)
                torch._foreach_mul_(vs, b2)
                torch._foreach_addcmul_(vs, gs, gs, value=1 - b2)
            bc1 = 1 - b1 ** self.step_id
            bc2 = 1 - b2 ** min(self.step_id, self.warmup_steps)
            denom = torch._foreach_sqrt(vs)
            torch._foreach_div_(denom, bc2 ** 0.5)
            torch._foreach_add_(denom, eps)
            torch._foreach_addcdiv_(ps, ms, denom, value=-lr / bc1)
        return loss


class QAdamAlgorithm(Algorithm):
    """Full-precision gradient all-reduce while the optimizer warms up, then compressed
    all-reduce of the momentum."""

    def __init__(self, q_adam_optimizer: QAdamOptimizer, hierarchical: bool = False):
        self.optimizer = q_adam_optimizer
        self.hierarchical = hierarchical
        self._compressed = False

    def _want_compressed(self):
        # `step_id` counts completed optimizer steps; the step being computed is step_id + 1
        return self.optimizer.step_id >= self.optimizer.warmup_steps

    def need_reset(self, bm):
        return self._want_compressed() != self._compressed

    def init_tensors(self, bm):
        self._compressed = self._want_compressed()
        if not self._compressed:
            return super().init_tensors(bm)
        tensors = []
        for name, p in reversed(bm._named_params):
            m = self.optimizer.state[p]["exp_avg"]
            tensors.append(BaguaTensor(m, name + ".exp_avg", owner=p, kind="momentum"))
        return tensors

    def init_operations(self, bm, bucket):
        bucket.clear_ops()
        if self._compressed:
            bucket.append_centralized_synchronous_op(bm.pg, hierarchical=self.hierarchical, average=True,
                                                     scattergather=True, compression="MinMaxUInt8")
        else:
            bucket.append_centralized_synchronous_op(bm.pg, hierarchical=self.hierarchical, average=True)

    def init_backward_hooks(self, bm):
        if not self._compressed:
            return super().init_backward_hooks(bm)
        hooks = []
        by_param = {id(t.owner): t for b in bm.bagua_buckets for t in b.tensors if t.owner is not None}
        b1 = self.optimizer.param_groups[0]["betas"][0]

        # m = b1 m + (1 - b1) g for a whole bucket at once, when its last gradient has arrived: two
        # multi-tensor launches per bucket instead of two small kernels per parameter.  Nothing is
        # lost by waiting, a bucket is only communicated once all of its tensors are ready.
        for b in bm.bagua_buckets:
            b._qadam_owned = sum(1 for t in b.tensors if t.owner is not None)
            b._qadam_arrived = []

        def make(t):
            def hook(param):
                if bm._in_no_sync:
                    return
                b = t._bucket
                b._qadam_arrived.append((t, param.grad))
                if len(b._qadam_arrived) < b._qadam_owned:
                    return
                arrived, b._qadam_arrived = b._qadam_arrived, []
                with torch.no_grad():
                    ms = [a.tensor for a, _ in arrived]
                    torch._foreach_mul_(ms, b1)
                    torch._foreach_add_(ms, [g for _, g in arrived], alpha=1 - b1)
                for a, _ in arrived:
                    bm.mark_ready(a)

            return hook

        for _, p in bm._named_params:
            t = by_param.get(id(p))
            if t is not None:
                hooks.append(p.register_post_accumulate_grad_hook(make(t)))
        return hooks

    def flush_unready(self, bm):
        if self._compressed:
            # buckets with some gradients missing: update the momentum of those that did arrive
            b1 = self.optimizer.param_groups[0]["betas"][0]
            for b in bm.bagua_buckets:
                arrived, b._qadam_arrived = getattr(b, "_qadam_arrived", []), []
                if arrived:
                    with torch.no_grad():
                        ms = [a.tensor for a, _ in arrived]
                        torch._foreach_mul_(ms, b1)
                        torch._foreach_add_(ms, [g for _, g in arrived], alpha=1 - b1)
                    for a, _ in arrived:
                        bm.mark_ready(a)
        bm.flush_unready()

    def state_dict(self, bm):
        return {"compressed": self._compressed}


class AsyncModelAverageAlgorithm(_WeightAlgorithm):
    """Asynchronous model averaging: a background thread all-reduces the weights every
    `sync_interval_ms` while training continues; the delta is applied with atomics.
    `abort(bm)` stops it (e.g. before evaluation), `resume(bm)` restarts it.

    Every rank's thread runs on its own timer, but an averaging round is a collective: before each
    round the threads agree (one small host all-reduce on a control group of their own) whether any
    rank has asked to stop.  If one has, no rank starts the round and every rank's thread ends, so a
    rank that stops first never leaves its peers waiting inside a round for it.  `abort` is therefore
    collective in effect (the first rank to call it stops averaging everywhere), and `resume` must be
    called on every rank."""

    def __init__(self, peer_selection_mode: str = "all", sync_interval_ms: int = 500, warmup_steps: int = 0):
        assert peer_selection_mode == "all"
        self.peer_selection_mode = peer_selection_mode
        self.sync_interval_ms = sync_interval_ms
        self.warmup_steps = warmup_steps
        self._thread = None
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self._ctl_group = None  # host-side group on which the threads agree to go on or to stop
        self.rounds = 0

    def tensors_to_buckets(self, bm, tensors):
        return [list(tensors)]  # one bucket: the whole model is averaged at once

    def init_operations(self, bm, bucket):
        import torch.distributed as dist

        if self._ctl_group is None and bm.pg.world_size > 1:
            # collective: every rank builds its buckets at the same point of `with_bagua`
            self._ctl_group = dist.new_group(backend="gloo")
        bucket.clear_ops()
        if bm.bagua_train_step_counter < self.warmup_steps:
            bucket.append_centralized_synchronous_op(bm.pg, hierarchical=False, average=True)
        else:
            bucket.append_asynchronous_model_average_op(bm.pg, self.peer_selection_mode)

    def need_reset(self, bm):
        return self.warmup_steps > 0 and bm.bagua_train_step_counter == self.warmup_steps

    def init_forward_pre_hooks(self, bm):
        def pre(_module, _inputs):
            if bm.bagua_train_step_counter >= self.warmup_steps and self._thread is None and not self._stop.is_set():
                self._start(bm)

        return [bm.module.register_forward_pre_hook(pre)]

    def init_post_backward_hook(self, bm):
        def hook():
            if bm.bagua_train_step_counter < self.warmup_steps:
                self._mark_all(bm)
                bm.pg.backend.wait_pending_comm_ops()
                bm.pg.wait_comm_stream()

        return hook

    def _loop(self, bm):
        if bm.pg.is_cuda:
            torch.cuda.set_device(bm.pg.device)
        import torch.distributed as dist

        while True:
            self._stop.wait(self.sync_interval_ms / 1000.0)
            with self._lock:
                if self._ctl_group is not None:
                    # does any rank want to stop?  All ranks get the same answer, so all go on or all leave.
                    flag = torch.tensor([1 if self._stop.is_set() else 0], dtype=torch.int32)
                    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self._ctl_group)
                    if int(flag.item()):
                        self._stop.set()
                        break
                elif self._stop.is_set():
                    break
                for b in bm.bagua_buckets:
                    for t in b.tensors:
                        bm.pg.backend.mark_communication_ready(t.backend_tensor, 0)
                bm.pg.backend.wait_pending_comm_ops()
                self.rounds += 1

    def _start(self, bm):
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, args=(bm,), daemon=True, name="bagua-async-average")
        self._thread.start()

    def abort(self, bm):
        """Stop averaging; returns once no averaging round is in flight on this rank.  The other ranks'
        threads learn of it at their next round and stop as well."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def resume(self, bm):
        """Restart averaging; call it on every rank."""
        if self._thread is not None and not self._thread.is_alive():
            self._thread.join()
            self._thread = None
        if self._thread is None:
            self._start(bm)
