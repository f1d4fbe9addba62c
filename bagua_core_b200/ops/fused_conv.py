"""Convolution block with the element-wise tail fused: conv → (bias + ReLU) in one in-place pass,
and in the backward one pass that applies the ReLU mask and reduces the bias gradient.

The convolution itself stays a library call (cuDNN through `aten.convolution` /
`aten.convolution_backward`).  What the framework would run around it — a bias add, a clamp, a
ReLU-mask kernel and a separate column reduction for the bias gradient — is replaced by the two
sm_100a kernels of `csrc/kernels/model_ops.cu`.  The fused path needs a block computed in bf16
(bf16 autocast on CUDA, or bf16 parameters and inputs); anything else takes the plain PyTorch
composition, so `ConvBiasReLU` is a drop-in for `Conv2d` followed by `ReLU`.  bf16 tensors on the
CPU run the same Python path against a host restatement of the kernels
(`csrc/kernels/model_ops_cpu.cc`), which is how the glue is tested without a GPU.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._native import C as _C
from . import shadow as _shadow


# Kernels of this module launched so far in this process (benchmarks report it).
launches = 0


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream if t.is_cuda else 0


def _count(n: int) -> None:
    global launches
    launches += n


def _autocast_inputs(*tensors):
    """What an autocast-aware op does with its inputs: inside an autocast region of the tensors'
    device, floating-point inputs are cast to the region's dtype; elsewhere they pass through."""
    dev = tensors[0].device.type
    if not torch.is_autocast_enabled(dev):
        return tensors
    dtype = torch.get_autocast_dtype(dev)
    return tuple(t.to(dtype) if t.is_floating_point() else t for t in tensors)


def _autocast_weight(weight: torch.Tensor) -> torch.Tensor:
    """The weight in the autocast dtype; taken from the optimizer's bf16 copy when that is current
    (`bagua_core_b200.ops.shadow`), so that the forward pass does not cast it again."""
    dev = weight.device.type
    if not torch.is_autocast_enabled(dev):
        return weight
    return _shadow.cast_weight(weight, torch.get_autocast_dtype(dev))


class _ConvBiasReLUFn(torch.autograd.Function):
    """Runs in the autocast dtype where autocast is on (parameters stay fp32 outside; autograd
    casts the gradients returned here back to the parameters' dtype)."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation, groups):
        ctx.conf = (stride, padding, dilation, groups)
        x, bias = _autocast_inputs(x, bias)
        weight = _autocast_weight(weight)
        with torch.autocast(x.device.type, enabled=False):
            x = x.contiguous(memory_format=torch.channels_last)
            z = torch.ops.aten.convolution(x, weight, None, stride, padding, dilation, False, [0, 0], groups)
            z = z.contiguous(memory_format=torch.channels_last)
        _C.k_bias_relu_(z, bias.contiguous(), _stream(z))
        _count(1)
        ctx.save_for_backward(x, weight, z)
        return z

    @staticmethod
    def backward(ctx, dy):
        stride, padding, dilation, groups = ctx.conf
        x, weight, y = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dz = torch.empty_like(y)
        db = torch.empty(weight.shape[0], dtype=torch.float32, device=y.device)
        _C.k_bias_relu_backward(dy, y, dz, db, _stream(y))
        _count(2)  # mask + partial sums, then the fold of the partial sums
        with torch.autocast(y.device.type, enabled=False):
            dx, dw, _ = torch.ops.aten.convolution_backward(
                dz, x, weight, None, stride, padding, dilation, False, [0, 0], groups,
                [ctx.needs_input_grad[0], ctx.needs_input_grad[1], False])
        return dx, dw, db, None, None, None, None  # fp32; autograd casts it to the bias parameter's dtype


class _ConvBiasReLUPoolFn(torch.autograd.Function):
    """conv → bias + ReLU → 2x2 max pooling; the full-resolution activation is kept only for the
    backward, which produces the convolution's output gradient and the bias gradient in one pass."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation, groups):
        ctx.conf = (stride, padding, dilation, groups)
        x, bias = _autocast_inputs(x, bias)
        weight = _autocast_weight(weight)
        with torch.autocast(x.device.type, enabled=False):
            x = x.contiguous(memory_format=torch.channels_last)
            y = torch.ops.aten.convolution(x, weight, None, stride, padding, dilation, False, [0, 0], groups)
            y = y.contiguous(memory_format=torch.channels_last)
        n, c, h, w = y.shape
        p = torch.empty((n, c, h // 2, w // 2), dtype=y.dtype, device=y.device, memory_format=torch.channels_last)
        _C.k_bias_relu_pool_(y, p, bias.contiguous(), _stream(y))
        _count(1)
        ctx.save_for_backward(x, weight, y)
        return p

    @staticmethod
    def backward(ctx, dp):
        stride, padding, dilation, groups = ctx.conf
        x, weight, y = ctx.saved_tensors
        dp = dp.contiguous(memory_format=torch.channels_last)
        dz = torch.empty_like(y)
        db = torch.empty(weight.shape[0], dtype=torch.float32, device=y.device)
        _C.k_bias_relu_pool_backward(dp, y, dz, db, _stream(y))
        _count(2)
        with torch.autocast(y.device.type, enabled=False):
            dx, dw, _ = torch.ops.aten.convolution_backward(
                dz, x, weight, None, stride, padding, dilation, False, [0, 0], groups,
                [ctx.needs_input_grad[0], ctx.needs_input_grad[1], False])
        return dx, dw, db, None, None, None, None  # fp32; autograd casts it to the bias parameter's dtype


class _MaxPool2x2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        y = torch.empty((n, c, h // 2, w // 2), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        _C.k_maxpool2x2_forward(x, y, _stream(x))
        _count(1)
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty_like(x, memory_format=torch.channels_last)
        _C.k_maxpool2x2_backward(x, dy, dx, _stream(x))
        _count(1)
        return dx


class MaxPool2x2(nn.Module):
    """`nn.MaxPool2d(2, 2)`.  Channels-last CUDA bf16 inputs with even height and width go through
    this package's kernels: no index tensor in the forward, and a backward that recomputes the
    arg-max and writes the whole input gradient in one pass (no zero-fill)."""

    def forward(self, x):
        if (x.dtype == torch.bfloat16 and x.dim() == 4
                and x.is_contiguous(memory_format=torch.channels_last)
                and _C.k_maxpool2x2_supported(x.shape[0], x.shape[2], x.shape[3], x.shape[1])):
            return _MaxPool2x2Fn.apply(x)
        return F.max_pool2d(x, 2, 2)


def _computes_in_bf16(x: torch.Tensor, weight: torch.Tensor) -> bool:
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type) == torch.bfloat16
    return x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16


class ConvBiasReLU(nn.Conv2d):
    """`nn.Conv2d` (with bias) followed by ReLU, with the same parameters and state dict as the
    convolution alone."""

    def forward(self, x):
        fusable = (self.bias is not None and not isinstance(self.padding, str) and self.padding_mode == "zeros"
                   and x.dim() == 4 and _computes_in_bf16(x, self.weight)
                   and _C.k_bias_relu_supported(1, self.out_channels))
        if not fusable:
            return F.relu(super().forward(x))
        return _ConvBiasReLUFn.apply(x, self.weight, self.bias, list(self.stride), list(self.padding),
                                     list(self.dilation), self.groups)


class ConvBiasReLUPool(nn.Conv2d):
    """`nn.Conv2d` (with bias) followed by ReLU and `MaxPool2d(2, 2)`, with the convolution's
    parameters and state dict.  On the fused path the pooling is folded into the bias + ReLU pass
    in both directions, so the full-resolution activation is read once on the way forward and its
    gradient is written once on the way back."""

    def forward(self, x):
        fusable = (self.bias is not None and not isinstance(self.padding, str) and self.padding_mode == "zeros"
                   and x.dim() == 4 and _computes_in_bf16(x, self.weight)
                   and _C.k_bias_relu_supported(1, self.out_channels))
        if fusable:
            # the convolution's output size decides whether the 2x2 windows tile it exactly
            h = (x.shape[2] + 2 * self.padding[0] - self.dilation[0] * (self.kernel_size[0] - 1) - 1) // self.stride[0] + 1
            w = (x.shape[3] + 2 * self.padding[1] - self.dilation[1] * (self.kernel_size[1] - 1) - 1) // self.stride[1] + 1
            fusable = _C.k_maxpool2x2_supported(x.shape[0], h, w, self.out_channels)
        if not fusable:
            return F.max_pool2d(F.relu(super().forward(x)), 2, 2)
        return _ConvBiasReLUPoolFn.apply(x, self.weight, self.bias, list(self.stride), list(self.padding),
                                         list(self.dilation), self.groups)
