"""Optimizers that work on flat bucket memory with one fused kernel per bucket.

The reference contains no optimizer (it is only the communication engine); the benchmarks
named for it train with SGD momentum 0.9, so the engine ships the obvious companion: since
gradients already live in flat buckets, parameters and momentum are laid out the same way
and `step()` is ONE sm_100a kernel per bucket (read p, g, m; write p, m: 20 bytes per
parameter, the HBM minimum) instead of torch's multi-tensor loops.
"""
from __future__ import annotations

from typing import List

import torch

from .._native import C as _C


def _is_dense(t: torch.Tensor) -> bool:
    """True if the tensor's elements occupy one gap-free, non-overlapping block of memory."""
    if t.numel() <= 1:
        return True
    dims = sorted((st, sz) for st, sz in zip(t.stride(), t.shape) if sz > 1)
    expect = 1
    for st, sz in dims:
        if st != expect:
            return False
        expect *= sz
    return True


class FlatSGD(torch.optim.Optimizer):
    """torch.optim.SGD semantics (momentum, dampening, weight decay, Nesterov).

    Before `with_bagua` attaches it (or for parameters outside any bucket) it updates
    parameter by parameter with the same kernel.

    `bf16_shadow=True`: for buckets of gradients (algorithms that do not communicate weights) the
    step kernel also writes every updated parameter rounded to bf16 into a second flat buffer, and
    each parameter gets a view of it (`bagua_core_b200.ops.shadow`); `ConvBiasReLU`,
    `ConvBiasReLUPool` and `ShadowLinear` under bf16 autocast then read their weights from there
    instead of casting the fp32 master weights in every forward pass.  After changing a parameter
    by other means than this optimizer or torch's in-place ops, call `refresh_bf16()`."""

    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, bf16_shadow: bool = False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        defaults = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)
        super().__init__(params, defaults)
        self._flat: List[dict] = []
        self._attached_ids = set()
        self._steps = 0
        self.kernel_launches = 0
        # bf16 copies of the weights, written by the step kernel (see bagua_core_b200.ops.shadow)
        self.bf16_shadow = bf16_shadow
        self.shadows_valid = False
        self._shadowed: List[torch.Tensor] = []

    def _group_runs(self, bucket):
        """[(start, end, group index)] over a bucket's flat elements: maximal runs of consecutive
        parameters that belong to the same parameter group, so that each run is stepped with its own
        group's learning rate, momentum and weight decay.  With one group (or a bucket whose parameters
        all share a group) that is one run over the whole bucket, padding included."""
        group_of = {id(p): gi for gi, g in enumerate(self.param_groups) for p in g["params"]}
        runs, off = [], 0
        for t in bucket.tensors:
            n = t.owner.numel()
            gi = group_of.get(id(t.owner))
            if gi is None:
                raise RuntimeError(f"parameter of bucket tensor `{t.name}` is not in this optimizer")
            if runs and runs[-1][2] == gi:
                runs[-1][1] = off + n
            else:
                runs.append([off, off + n, gi])
            off += n
        if runs:
            runs[-1][1] = bucket.flattened.numel()  # the padding (zero gradient, zero weights) rides along
        return [tuple(r) for r in runs]

    # called by BaguaModule after it has built gradient buckets
    def bagua_attach(self, bm):
        self._flat.clear()
        self._attached_ids.clear()
        for p in self._shadowed:
            p._bagua_bf16 = None
        self._shadowed.clear()
        self.shadows_valid = False
        for b in bm.bagua_buckets:
            if b.flattened is not None and b.flattened.dtype == torch.float32 and all(
                    t.kind == "weight" for t in b.tensors):
                # weights are the bucket: give the gradients the same flat layout
                flat_g = torch.zeros_like(b.flattened)
                off = 0
                for t in b.tensors:
                    p = t.owner
                    n = p.numel()
                    p.grad = flat_g[off:off + n].as_strided(tuple(p.shape), tuple(p.stride()))
                    self._attached_ids.add(id(p))
                    off += n
                self._flat.append({"p": b.flattened, "g": flat_g, "m": torch.zeros_like(flat_g), "first": True,
                                   "runs": self._group_runs(b)})
                continue
            if b.flattened is None or any(t.kind != "grad" for t in b.tensors):
                continue
            if b.flattened.dtype != torch.float32:
                continue
            flat_p = torch.zeros_like(b.flattened)
            off = 0
            with torch.no_grad():
                for t in b.tensors:
                    p = t.owner
                    n = p.numel()
                    shape, stride = tuple(p.shape), tuple(p.stride())
                    if tuple(t.tensor.stride()) != stride:
                        raise RuntimeError("parameter and gradient layouts differ; cannot share a flat layout")
                    flat_p[off:off + n].as_strided(shape, stride).copy_(p)
                    p.set_(flat_p.untyped_storage(), off, shape, stride)
                    self._attached_ids.add(id(p))
                    off += n
            entry = {"p": flat_p, "g": b.flattened, "m": torch.zeros_like(flat_p), "first": True,
                     "runs": self._group_runs(b)}
            if self.bf16_shadow:
                from ..ops.shadow import BF16Shadow

                flat_h = torch.zeros_like(flat_p, dtype=torch.bfloat16)
                off = 0
                for t in b.tensors:
                    p = t.owner
                    n = p.numel()
                    p._bagua_bf16 = BF16Shadow(flat_h[off:off + n].as_strided(tuple(p.shape), tuple(p.stride())), self)
                    self._shadowed.append(p)
                    off += n
                entry["h"] = flat_h
            self._flat.append(entry)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        stream = torch.cuda.current_stream().cuda_stream if (self._flat and self._flat[0]["p"].is_cuda) else 0
        for f in self._flat:
            # one launch per run of parameters that share a parameter group (usually one per bucket),
            # each with its own group's hyperparameters as they are now (schedulers change them in place)
            whole = len(f["runs"]) == 1
            for lo, hi, gi in f["runs"]:
                g = self.param_groups[gi]
                p_, g_, m_ = (f["p"], f["g"], f["m"]) if whole else (f["p"][lo:hi], f["g"][lo:hi], f["m"][lo:hi])
                if "h" in f:
                    h_ = f["h"] if whole else f["h"][lo:hi]
                    _C.k_sgd_momentum_flat_shadow(p_, g_, m_, h_, g["lr"], g["momentum"], g["dampening"],
                                                  g["weight_decay"], g["nesterov"], f["first"], stream)
                else:
                    _C.k_sgd_momentum_flat(p_, g_, m_, g["lr"], g["momentum"], g["dampening"], g["weight_decay"],
                                           g["nesterov"], f["first"], stream)
                self.kernel_launches += 1
            f["first"] = False
        if self._shadowed and not self.shadows_valid:
            self._validate_shadows()
        for group in self.param_groups:
            for p in group["params"]:
                if id(p) in self._attached_ids or p.grad is None:
                    continue
                st = self.state[p]
                first = "momentum_buffer" not in st
                if first:
                    st["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                buf = st["momentum_buffer"]
                same_layout = (p.dtype == torch.float32 and _is_dense(p) and p.grad.dtype == torch.float32
                               and p.grad.stride() == p.stride() and buf.stride() == p.stride())
                if not same_layout:
                    # layouts differ (e.g. autograd produced a contiguous gradient for a
                    # channels_last weight): element-wise torch math is layout-agnostic
                    d = p.grad.add(p, alpha=group["weight_decay"]) if group["weight_decay"] else p.grad
                    if group["momentum"]:
                        if first:
                            buf.copy_(d)
                        else:
                            buf.mul_(group["momentum"]).add_(d, alpha=1 - group["dampening"])
                        d = d.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    p.add_(d, alpha=-group["lr"])
                    continue
                s = torch.cuda.current_stream().cuda_stream if p.is_cuda else 0
                # dense tensors with equal strides can be updated as flat memory
                pv = torch.as_strided(p, (p.numel(),), (1,))
                gv = torch.as_strided(p.grad, (p.numel(),), (1,))
                mv = torch.as_strided(st["momentum_buffer"], (p.numel(),), (1,))
                _C.k_sgd_momentum_flat(pv, gv, mv, group["lr"], group["momentum"], group["dampening"],
                                       group["weight_decay"], group["nesterov"], first, s)
                self.kernel_launches += 1
        self._steps += 1
        return loss

    def _validate_shadows(self):
        """The bf16 copies equal the parameters now: remember the parameters' versions."""
        for p in self._shadowed:
            p._bagua_bf16.version = p._version
        self.shadows_valid = True

    @torch.no_grad()
    def refresh_bf16(self):
        """Recomputes the bf16 copies from the parameters (after the weights were changed by something
        the copies cannot notice, or to use them before the first step)."""
        for f in self._flat:
            if "h" in f:
                f["h"].copy_(f["p"])
        if self._shadowed:
            self._validate_shadows()

    def zero_grad(self, set_to_none: bool = False):
        """Zero the flat gradient buffers with one memset per bucket; gradients stay views
        of the bucket (never set to None, which would detach them from the bucket)."""
        for f in self._flat:
            f["g"].zero_()
        for group in self.param_groups:
            for p in group["params"]:
                if id(p) not in self._attached_ids and p.grad is not None:
                    p.grad.zero_()
