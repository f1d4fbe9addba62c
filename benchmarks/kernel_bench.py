#!/usr/bin/env python
"""Single-GPU roofline check of the engine's streaming kernels.

    python benchmarks/kernel_bench.py [--mb 256] [--only sgd,compress,...] [--iters 10] [--json out.json]

Each kernel runs on inputs larger than the 126 MB L2 (default 256 MB of fp32 per operand),
is timed with CUDA events after warm-up with an L2 flush before every timed launch, and is
reported as algorithmic bytes / time against the measured HBM copy bandwidth
(`MEASURED_PEAKS.json`, "of measured"; the documented fallback otherwise, "of fallback").
`--iters 1 --warmup 1 --only X` gives a short run suitable for an `ncu` capture.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bagua_core as bc  # noqa: E402
import bagua_core_b200.ops as ops  # noqa: E402
from bagua_core_b200.utils import flush_l2, load_measured_peaks  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    n = args.mb * (1 << 20) // 4
    peaks = load_measured_peaks()
    hbm = peaks["hbm_gbs"]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, generator=g).cuda()
    y = torch.randn(n, generator=g).cuda()
    m = torch.zeros_like(x)
    S = n * 4
    n_chunks = 8
    bx = bc.BaguaTensorPy(x, "x")
    comp = bx.compress("MinMaxUInt8", n_chunks, -1)
    out = torch.empty_like(x)
    bo = bc.BaguaTensorPy(out, "o")

    cases = {
        # name: (callable, algorithmic bytes)
        "add": (lambda: ops.add_inplace(x, y), 3 * S),
        "addmul": (lambda: ops.addmul_inplace(x, y, 0.5), 3 * S),
        "average": (lambda: ops.average_inplace(x, y), 3 * S),
        "divide": (lambda: ops.divide_inplace(x, 1.0001), 2 * S),
        "reduce_chunk": (lambda: ops.reduce_chunk_inplace(x, n_chunks, 0, average=True), S + S // n_chunks),
        "async_average": (lambda: ops.async_model_average(x, y, m, 8), 4 * S),
        "sgd": (lambda: ops.sgd_momentum_flat(x, y, m, 1e-6, 0.9), 5 * S),
        # two passes over the input (min/max, then quantise) + 1 byte per element out
        "compress": (lambda: bx.compress("MinMaxUInt8", n_chunks, -1), 2 * S + S // 4),
        "decompress": (lambda: bo.decompress_from("MinMaxUInt8", n_chunks, comp), S // 4 + S),
    }
    only = [s for s in args.only.split(",") if s]
    rows = []
    for name, (fn, nbytes) in cases.items():
        if only and name not in only:
            continue
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.iters):
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        ms = times[len(times) // 2]
        gbs = nbytes / (ms * 1e-3) / 1e9
        row = {"kernel": name, "mb_per_operand": args.mb, "ms": ms, "algorithmic_gb": nbytes / 1e9, "gbs": gbs,
               "frac_of_hbm": gbs / hbm, "peak_source": peaks["source"], "hbm_gbs": hbm}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
