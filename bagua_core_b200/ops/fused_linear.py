"""`nn.Linear` that reads its weight from the optimizer's bf16 copy.

Drop-in for `nn.Linear`: unless an optimizer maintains a bf16 copy of the weight
(`bagua_core_b200.ops.shadow`) and the call is inside a bf16 autocast region, it is `nn.Linear`.
Otherwise forward and backward run the same
three GEMMs as the framework's own bf16 linear layer — y = x Wᵀ + b, dx = dy W, dW = dyᵀ x, library
calls — but on the optimizer's copy of W instead of a fresh cast of the fp32 master weight (for
VGG-16's first classifier layer alone that cast moves 0.6 GB per step).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import shadow as _shadow


class _ShadowLinearFn(torch.autograd.Function):
    """`weight` is the fp32 parameter (it receives the gradient); `w` its current bf16 copy."""

    @staticmethod
    def forward(ctx, x, weight, bias, w):
        x = x.to(torch.bfloat16)
        b = bias.to(torch.bfloat16) if bias is not None else None
        with torch.autocast(x.device.type, enabled=False):
            y = F.linear(x, w, b)
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
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
                dw = dy2.t() @ x.reshape(-1, x.shape[-1])  # bf16; autograd casts it to the parameter's dtype
            if ctx.has_bias and ctx.needs_input_grad[2]:
                db = dy2.sum(0, dtype=torch.float32)
        return dx, dw, db, None


class ShadowLinear(nn.Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dev = x.device.type
        managed = getattr(self.weight, "_bagua_bf16", None) is not None  # an optimizer keeps a bf16 copy
        if managed and torch.is_autocast_enabled(dev) and torch.get_autocast_dtype(dev) == torch.bfloat16:
            # the copy when it is current, a fresh cast otherwise: the same code path either way
            return _ShadowLinearFn.apply(x, self.weight, self.bias, _shadow.cast_weight(self.weight, torch.bfloat16))
        return super().forward(x)
