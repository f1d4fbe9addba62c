"""`nn.Linear` that reads its weight from the optimizer's bf16 copy.

Drop-in for `nn.Linear`: unless the call is inside a bf16 autocast region and either an optimizer
maintains a bf16 copy of the weight (`bagua_core_b200.ops.shadow`) or in-place weight-gradient
accumulation is switched on (`bagua_core_b200.ops.wgrad`), it is `nn.Linear`.
Otherwise forward and backward run the same
three GEMMs as the framework's own bf16 linear layer — y = x Wᵀ + b, dx = dy W, dW = dyᵀ x, library
calls — but on the optimizer's copy of W instead of a fresh cast of the fp32 master weight (for
VGG-16's first classifier layer alone that cast moves 0.6 GB per step), and, with `wgrad.enabled`,
with the dW GEMM adding its product straight into the fp32 `weight.grad` instead of handing a bf16
matrix to autograd for a cast and a separate accumulation.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import shadow as _shadow
from . import wgrad as _wgrad


class _ShadowLinearFn(torch.autograd.Function):
    """`weight` is the fp32 parameter (it receives the gradient); `w` its current bf16 copy or a fresh
    cast; `owner` the module, through which backward reaches the parameter object itself (its `.grad`
    and hooks) when it accumulates the weight gradient in place."""

    @staticmethod
    def forward(ctx, x, weight, bias, w, owner):
        x = x.to(torch.bfloat16)
        b = bias.to(torch.bfloat16) if bias is not None else None
        with torch.autocast(x.device.type, enabled=False):
            y = F.linear(x, w, b)
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.owner = owner
        ctx.use = _wgrad.begin_use(owner.weight) if (_wgrad.enabled and weight.requires_grad) else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = db = None
        with torch.autocast(dy.device.type, enabled=False):
            dy2 = dy.reshape(-1, dy.shape[-1])
            if ctx.needs_input_grad[0]:
                dx = (dy2 @ w).view(x.shape)
            if ctx.needs_input_grad[1]:
                x2 = x.reshape(-1, x.shape[-1])
                if not _wgrad.accumulate(ctx.owner.weight, ctx.use, dy2, x2):
                    dw = dy2.t() @ x2  # bf16; autograd casts it to the parameter's dtype
            if ctx.has_bias and ctx.needs_input_grad[2]:
                db = dy2.sum(0, dtype=torch.float32)
        return dx, dw, db, None, None


class ShadowLinear(nn.Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dev = x.device.type
        managed = getattr(self.weight, "_bagua_bf16", None) is not None  # an optimizer keeps a bf16 copy
        if ((managed or _wgrad.enabled) and torch.is_autocast_enabled(dev)
                and torch.get_autocast_dtype(dev) == torch.bfloat16):
            # the copy when it is current, a fresh cast otherwise: the same code path either way
            return _ShadowLinearFn.apply(x, self.weight, self.bias, _shadow.cast_weight(self.weight, torch.bfloat16),
                                         self)
        return super().forward(x)
