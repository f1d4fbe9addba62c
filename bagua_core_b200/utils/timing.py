"""Device-side timing helpers (CUDA events on the launching stream) and roofline peaks."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

import torch

_FLUSH = {}


def flush_l2(device=None):
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    device = device or torch.cuda.current_device()
    buf = _FLUSH.get(device)
    if buf is None:
        buf = _FLUSH[device] = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device)
    buf.zero_()


def cuda_time_ms(fn: Callable[[], None], iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    """Median device time of `fn` in ms over `iters` runs, each bracketed by events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def load_measured_peaks(repo_root: str = None) -> Dict:
    """Roofline denominators: the measured figures if the file is present, else the
    documented fallback (marked as such)."""
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
