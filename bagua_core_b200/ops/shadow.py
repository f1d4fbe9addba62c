"""bf16 copies of fp32 master weights, kept current by the optimizer.

Under bf16 autocast every forward pass casts every fp32 weight to bf16 again (for VGG-16 that is
33 cast kernels and 0.8 GB of traffic per step, about 5 % of the step on a B200).  An optimizer
that already streams over all parameters can write the bf16 value of each updated parameter in the
same pass (`FlatSGD(bf16_shadow=True)`, kernel `sgd_shadow_kernel` in `csrc/kernels/elementwise.cu`);
modules that compute in bf16 then take their weight from that copy (`lookup`) and skip the cast.

A copy is used only while it is known to equal the parameter rounded to bf16:

* the owner (the optimizer) has marked its copies valid (after its first step, or `refresh_bf16()`),
* the parameter's version counter still has the value recorded then (any in-place change made
  through torch — `load_state_dict`, `param.add_()`, ... — bumps it; the optimizer's own kernel
  does not).

A change that bypasses the counter (writing through `param.data`, a communication op that averages
weights) is invisible here: call the optimizer's `refresh_bf16()` after it.  `FlatSGD` does not hand
out copies for buckets whose algorithm communicates weights.
"""
from __future__ import annotations

from typing import Optional

import torch

# False: every lookup misses, so modules cast as if no copies existed (tests compare the two).
enabled = True

# How often a module found a valid copy / had to cast (benchmarks and tests read these).
hits = 0
misses = 0


class BF16Shadow:
    """Attached to a parameter as `_bagua_bf16`."""

    __slots__ = ("view", "version", "owner")

    def __init__(self, view: torch.Tensor, owner):
        self.view = view        # bf16, same shape and strides as the parameter
        self.version = -1       # parameter version at which the copy was last known to be current
        self.owner = owner      # has `.shadows_valid`


def lookup(param: torch.Tensor) -> Optional[torch.Tensor]:
    """The current bf16 copy of `param`, or None."""
    s = getattr(param, "_bagua_bf16", None)
    if s is None or not enabled or not s.owner.shadows_valid or s.version != param._version:
        return None
    return s.view


def cast_weight(param: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """`param.to(dtype)`, without the cast when a current bf16 copy exists."""
    global hits, misses
    if dtype == torch.bfloat16 and param.dtype == torch.float32:
        v = lookup(param)
        if v is not None:
            hits += 1
            return v
        misses += 1
    return param.to(dtype)
