"""Python entry points of the tensor kernels (sm_100a on CUDA tensors, C++ loops on CPU
tensors).  All run on the current CUDA stream unless `stream` (a torch.cuda.Stream) is given.

Reference kernels: bagua-core-internal/kernels/bagua_kernels.cu:196-266 (element-wise,
async average), 373-400 (chunk reduce), 455-500 (MinMaxUInt8).
"""
from __future__ import annotations

import torch

from .._native import C as _C
from .. import BaguaTensorPy


def _s(t: torch.Tensor, stream=None) -> int:
    if not t.is_cuda:
        return 0
    return (stream or torch.cuda.current_stream(t.device)).cuda_stream


def divide_inplace(x, divisor, stream=None):
    _C.k_divide_inplace(x, float(divisor), _s(x, stream))
    return x


def add_inplace(x, y, stream=None):
    _C.k_add_inplace(x, y, _s(x, stream))
    return x


def subtract_inplace(x, y, stream=None):
    _C.k_subtract_inplace(x, y, _s(x, stream))
    return x


def addmul_inplace(x, y, factor, stream=None):
    _C.k_addmul_inplace(x, y, float(factor), _s(x, stream))
    return x


def average_inplace(x, y, stream=None):
    _C.k_average_inplace(x, y, _s(x, stream))
    return x


def async_model_average(t, reduced, copy, nranks, stream=None):
    _C.k_async_model_average(t, reduced, copy, float(nranks), _s(t, stream))
    return t


def reduce_chunk_inplace(x, n_chunks, target_chunk, average=True, stream=None):
    _C.k_reduce_chunk_inplace(x, int(n_chunks), int(target_chunk), bool(average), _s(x, stream))
    return x


def compress_minmax_uint8(x: torch.Tensor, n_chunks: int = 1, target_chunk: int = -1) -> BaguaTensorPy:
    """Returns the engine-owned compressed buffer (`to_numpy_u8()` reads it back).  Runs on
    the legacy default stream, like `BaguaTensorPy.compress`."""
    return BaguaTensorPy(x, "compress_input").compress("MinMaxUInt8", n_chunks, target_chunk)


def decompress_minmax_uint8(out: torch.Tensor, compressed: BaguaTensorPy, n_chunks: int = 1):
    BaguaTensorPy(out, "decompress_output").decompress_from("MinMaxUInt8", n_chunks, compressed)
    return out


def sgd_momentum_flat(p, g, buf, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                      first_step=False, stream=None):
    _C.k_sgd_momentum_flat(p, g, buf, lr, momentum, dampening, weight_decay, nesterov, first_step, _s(p, stream))
    return p
