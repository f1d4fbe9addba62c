#!/usr/bin/env python
"""Config 1 on the CPU backend: two ranks (gloo), one bucket of three fp32 tensors
([1024,1024], [4096], [512,256], N(0,1) from seed=rank), gradient all-reduce and ByteGrad
through the public bucket API.  Checks the results against the fp32 mean and prints wall-clock
time per bucket (the CPU backend is the correctness oracle and the timed CPU baseline).

    python benchmarks/cpu_config1.py
"""
from __future__ import annotations

import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

SHAPES = [(1024, 1024), (4096,), (512, 256)]


def worker(rank, world, iters):
    import torch.distributed as dist

    import bagua_core as bc

    comm = bc.BaguaSingleCommunicatorPy(rank, world, -1, 0, "c10d:" + dist.group.WORLD.group_name)
    backend = bc.BaguaCommBackendPy(100, -1)
    g = torch.Generator().manual_seed(rank)
    total = sum(int(np.prod(s)) for s in SHAPES)
    flat = torch.empty(total)
    views, off = [], 0
    for s in SHAPES:
        n = int(np.prod(s))
        v = flat[off:off + n].view(*s)
        v.copy_(torch.randn(*s, generator=g))
        views.append(v)
        off += n
    orig = flat.clone()
    out = {}
    for algo in ("gradient_allreduce", "bytegrad"):
        ts = [bc.BaguaTensorPy(v, f"{algo}_{i}") for i, v in enumerate(views)]
        bucket = bc.BaguaBucketPy(algo, ts)
        if algo == "gradient_allreduce":
            bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
        else:
            bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=True,
                                                     compression="MinMaxUInt8")
        backend.register_ordered_buckets([bucket])
        times = []
        for it in range(iters):
            flat.copy_(orig)
            dist.barrier()
            t0 = time.perf_counter()
            for t in ts:
                backend.mark_communication_ready(t, 0)
            backend.wait_pending_comm_ops()
            times.append(time.perf_counter() - t0)
        out[algo] = (flat.clone(), sorted(times)[len(times) // 2])
    backend.close()
    return orig, out


def main():
    from mp_util import run_ranks

    world, iters = 2, 7
    res = run_ranks(worker, world, args=(iters,))
    mean = sum(r[0] for r in res) / world
    ar, t_ar = res[0][1]["gradient_allreduce"]
    bg, t_bg = res[0][1]["bytegrad"]
    exact = bool(torch.equal(ar, mean))
    chunk = mean.numel() // world
    worst = 0.0
    for c in range(world):
        sl = slice(c * chunk, (c + 1) * chunk)
        rng = max((r[0][sl].max() - r[0][sl].min()).item() for r in res)
        worst = max(worst, (bg[sl] - mean[sl]).abs().max().item() / (2 * rng / 255))
    print(json.dumps({"config": "cpu world_size=2 gloo, bucket of 3 fp32 tensors (4.7 MB)",
                      "allreduce_exact": exact, "allreduce_ms": t_ar * 1e3,
                      "bytegrad_error_over_bound": worst, "bytegrad_ms": t_bg * 1e3,
                      "bucket_bytes": mean.numel() * 4}))
    return 0 if exact and worst <= 1.0 else 1


if __name__ == "__main__":
    sys.exit(main())
