#!/usr/bin/env python
"""Fused communication kernels on ONE GPU through the single-launch emulation.

    python benchmarks/emulated_fused_bench.py [--ranks 8] [--mb 64] [--only bytegrad] [--iters 5]

All virtual ranks live on GPU 0, so "peer" traffic is HBM traffic: the numbers say how
fast the kernels' own loops are (their HBM-side roofline), not how fast NVLink is.  The
script exists so that a fused kernel can be timed and captured by `ncu` from a single
process, e.g. (after the same command line has exited 0 without ncu):

    ncu --set full --clock-control none -k regex:bytegrad_emu_kernel -c 1 \
        -o prof_bytegrad_emu python benchmarks/emulated_fused_bench.py --only bytegrad --iters 1 --warmup 1

Per-rank buffers default to 64 MB of fp32 (8 ranks: 512 MB of buckets plus staging, larger
than the 126 MB L2, a few GB in total).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bagua_core_b200 as bb  # noqa: E402
from bagua_core_b200.utils import flush_l2, load_measured_peaks  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--mb", type=int, default=64, help="MB of fp32 per rank")
    ap.add_argument("--blocks", type=int, default=16, help="CTAs per virtual rank (ranks*blocks must be co-resident)")
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    N = args.ranks
    n = args.mb * (1 << 20) // 4 // (16 * N) * (16 * N)
    S = n * 4
    arena = bb._C.EmulatedArena(N, 0, 3 * S + (8 << 20))
    arena.set_deadline_ms(10000.0)
    hbm = load_measured_peaks()["hbm_gbs"]
    xs = [torch.randn(n, generator=torch.Generator().manual_seed(r)).cuda() for r in range(N)]
    aux = [[x.clone() for x in xs] for _ in range(3)]

    # algorithmic HBM bytes per call, summed over all virtual ranks (every "remote" access is local here)
    cases = {
        "allreduce_oneshot": (lambda: arena.allreduce(xs, xs, True, "oneshot", args.blocks), N * (N + 1 + N) * S),
        "allreduce_twoshot": (lambda: arena.allreduce(xs, xs, True, "twoshot", args.blocks), N * 6 * S),
        "allreduce_symmetric": (lambda: arena.allreduce(xs, xs, True, "symmetric", args.blocks), N * 2 * S),
        "allreduce_symmetric_tma": (lambda: arena.allreduce(xs, xs, True, "symmetric_tma", args.blocks), N * 2 * S),
        "bytegrad": (lambda: arena.bytegrad(xs, True, args.blocks), int(N * 3.75 * S)),
        "lp_ring": (lambda: arena.lp_ring(xs, aux[0], aux[1], aux[2], args.blocks), int(N * 13.75 * S)),
    }

    def bytegrad_pipelined():
        # the variant that sends the reduced chunks back one destination at a time (read per call)
        os.environ["BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK"] = "0"
        try:
            arena.bytegrad(xs, True, args.blocks)
        finally:
            os.environ.pop("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", None)

    # one more pass over a quantised chunk per destination (S/4 per rank) than the default
    cases["bytegrad_pipelined"] = (bytegrad_pipelined, int(N * 4.0 * S))
    # the communicator's collectives: every rank's buffer of S bytes is cut in N chunks of c = S/N
    c = S // N
    parts = [x[:n // N] for x in xs]
    cases.update({
        "allgather": (lambda: arena.collective("allgather", parts, aux[0], blocks=args.blocks),
                      N * c * (4 * (N - 1) + 2)),
        "allgather_symmetric": (lambda: arena.collective("allgather", parts, aux[0], symmetric=True, blocks=args.blocks),
                                N * c * 2 * N),
        "alltoall": (lambda: arena.collective("alltoall", xs, aux[0], blocks=args.blocks), N * c * (4 * (N - 1) + 2)),
        "reduce_scatter": (lambda: arena.collective("reduce_scatter", xs, [a[:n // N] for a in aux[1]],
                                                    blocks=args.blocks), N * c * (3 * (N - 1) + 2)),
        "reduce_scatter_symmetric": (lambda: arena.collective("reduce_scatter", xs, [a[:n // N] for a in aux[1]],
                                                              symmetric=True, blocks=args.blocks), N * c * (N + 1)),
        "broadcast_twophase": (lambda: arena.collective("broadcast_twophase", [], aux[2], root=0, blocks=args.blocks),
                               (N - 1) * S * 2 + (N - 1) * c * 2 * (N - 1)),
    })
    only = [s for s in args.only.split(",") if s]
    for name, (fn, nbytes) in cases.items():
        if only and name not in only:
            continue
        if name == "allreduce_oneshot" and N * S > 3 * S + (8 << 20):
            continue  # one-shot staging is N*S per rank: only for small buffers
        for _ in range(args.warmup):
            fn()
        times = []
        for _ in range(args.iters):
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()  # synchronous: returns after the kernel finished
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        ms = times[len(times) // 2]
        print(json.dumps({"kernel": name, "virtual_ranks": N, "mb_per_rank": S >> 20, "blocks_per_rank": args.blocks,
                          "ms": ms, "hbm_gbs": nbytes / (ms * 1e-3) / 1e9,
                          "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm}), flush=True)


if __name__ == "__main__":
    main()
