"""Weight gradients accumulated by the GEMM that computes them.

Under bf16 autocast a linear layer's weight gradient takes three passes over memory: the GEMM
dW = dyᵀ x writes it in bf16, autograd casts it to the fp32 of the master weight, and the
accumulation step adds it to `weight.grad` (here a view of a flat gradient bucket).  That is 18
bytes of traffic per weight after the GEMM; for VGG-16, whose classifier holds 124 M of the model's
138 M parameters, about 2 GB per step.  The library GEMM can instead read and write the fp32
gradient itself (`C = A B + C` with bf16 A, B and fp32 C): 8 bytes per weight, no cast, no separate
accumulation, and the product is never rounded to bf16.

`accumulate(param, state, dy2, x2)` does that for a parameter whose `.grad` is an fp32 tensor and
returns True; the caller's backward then returns no gradient for the weight, so autograd has
nothing to cast or add.  The parameter's post-accumulate-grad hooks (which is how `with_bagua`
learns that a gradient is final) still run: autograd runs them when it reaches the parameter even
without a gradient, and where a torch version does not, `accumulate` runs them itself.  It returns False, and touches nothing, whenever that shortcut would change
what the user sees:

* the feature is off (`enabled`, default False), or a higher-order graph is being built;
* `.grad` is missing, not fp32, not contiguous or of another shape;
* the parameter has tensor hooks (`register_hook`), which autograd would apply to the gradient;
* the same weight takes part in the graph more than once (`UseState`): autograd would add the uses'
  gradients first and accumulate once, so both uses take the ordinary path.

Reference: the reference engine is told about finished gradients per tensor
(bagua-core-internal/src/lib.rs:300-319); how the trainer produces them is outside it.
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch

# Off by default.
enabled = False

# Which library call accumulates on CUDA: "addmm" (one GEMM reads and writes the fp32 gradient),
# "mm_add" (GEMM with fp32 output, then an in-place add) or "off" (neither is available: callers
# fall back to returning the gradient).  Decided by the first call that runs on a GPU.
cuda_mode: Optional[str] = None

# Gradients accumulated in place so far / calls that declined (tests and benchmarks read these).
accumulated = 0
declined = 0


class UseState:
    """One use of a weight in a graph.  The function's context holds it strongly, the parameter
    weakly: while an earlier use of the same weight is still waiting for its backward, a new use
    marks both as shared, and neither accumulates in place."""

    __slots__ = ("shared", "done", "__weakref__")

    def __init__(self):
        self.shared = False
        self.done = False


def begin_use(param: torch.Tensor) -> UseState:
    """Call in the forward pass, once per use of `param`."""
    st = UseState()
    ref = getattr(param, "_bagua_wgrad_use", None)
    prev = ref() if ref is not None else None
    if prev is not None and not prev.done:
        prev.shared = True
        st.shared = True
    param._bagua_wgrad_use = weakref.ref(st)
    return st


def _gemm_into(grad: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> bool:
    """grad += dy2ᵀ x2 (fp32 accumulation of low-precision operands).  False if no in-place form
    is available on this device, in which case `grad` is unchanged."""
    global cuda_mode
    if not grad.is_cuda:
        # host: there is no mixed-precision GEMM; widen the operands (tests, CPU training)
        grad.addmm_(dy2.t().to(grad.dtype), x2.to(grad.dtype))
        return True
    a = dy2.t()
    if cuda_mode in (None, "addmm"):
        try:
            torch.addmm(grad, a, x2, out_dtype=torch.float32, out=grad)
            cuda_mode = "addmm"
            return True
        except (RuntimeError, TypeError, NotImplementedError):
            if cuda_mode == "addmm":
                raise  # it worked before: a real error, not a missing overload
            cuda_mode = "mm_add"
    if cuda_mode == "mm_add":
        try:
            grad.add_(torch.mm(a, x2, out_dtype=torch.float32))
            return True
        except (RuntimeError, TypeError, NotImplementedError):
            cuda_mode = "off"
    return False


def accumulate(param: torch.Tensor, state: Optional[UseState], dy2: torch.Tensor, x2: torch.Tensor) -> bool:
    """Adds dy2ᵀ x2 ([out, in] from dy2 [rows, out] and x2 [rows, in]) to `param.grad` in place and
    runs the parameter's post-accumulate-grad hooks.  True: done, return no gradient for the weight.
    False: nothing was touched, compute and return the gradient as usual."""
    global accumulated, declined
    if state is not None:
        state.done = True
    grad = param.grad
    ok = (enabled and state is not None and not state.shared and not torch.is_grad_enabled()
          and grad is not None and grad.dtype == torch.float32 and grad.is_contiguous()
          and grad.shape == param.shape and grad.device == dy2.device
          and not getattr(param, "_backward_hooks", None))
    if ok:
        with torch.no_grad():
            ok = _gemm_into(grad, dy2, x2)
    if not ok:
        declined += 1
        return False
    accumulated += 1
    if not _autograd_runs_hooks_without_a_gradient():
        hooks = getattr(param, "_post_accumulate_grad_hooks", None)
        if hooks:
            for hook in list(hooks.values()):
                hook(param)
    return True


_hooks_run_anyway: Optional[bool] = None


def _autograd_runs_hooks_without_a_gradient() -> bool:
    """Whether autograd runs a parameter's post-accumulate-grad hooks when the backward of its only
    consumer returned None for it.  torch 2.11 does (the hooks then run when autograd reaches the
    parameter, once, however many uses it had); where it does not, `accumulate` runs them itself.
    Found out once, on a three-element graph on the host."""
    global _hooks_run_anyway
    if _hooks_run_anyway is None:
        fired = []

        class _Probe(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x, w):
                return x * w.detach()

            @staticmethod
            def backward(ctx, dy):
                return dy, None

        with torch.enable_grad():
            w = torch.nn.Parameter(torch.ones(3))
            w.grad = torch.zeros(3)
            handle = w.register_post_accumulate_grad_hook(lambda p: fired.append(1))
            x = torch.ones(3, requires_grad=True)
            _Probe.apply(x, w).sum().backward()
            handle.remove()
        _hooks_run_anyway = bool(fired)
    return _hooks_run_anyway
