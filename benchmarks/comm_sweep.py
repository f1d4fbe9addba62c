#!/usr/bin/env python
"""Communication-op microbenchmark: latency and bus bandwidth of every engine op, fused
kernels versus the library (NCCL) path that replays the reference's call sequence.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 benchmarks/comm_sweep.py --out sweep_8gpu.json

Ops: gradient_allreduce (O1, average), bytegrad (O2), shift_one (O3 pair average),
lp_ring (O4), qadam (the compressed all-reduce of a momentum buffer: the same op as
bytegrad), each on one fp32 bucket of 1 KB … 1 GB (powers of 4), values N(0,1) from seed=rank.  Every op runs through the public bucket API (`BaguaBucketPy.append_*_op`,
`mark_communication_ready`, `wait_pending_comm_ops`).  Timing: CUDA events on the
communication stream around `iters` back-to-back buckets after `warmup`, an L2 flush
(192 MB memset) before each timed batch, max over ranks.  `raw_nccl` is a bare
`ncclAllReduce` through the communicator for reference.  `allgather`, `alltoall`,
`reduce_scatter` and `broadcast` (not in the default list) time the communicator's own
collectives on a buffer of the given total size, as peer-memory kernels (path `fused`) or
library calls (path `library`), issued from a Python op inside a bucket.  Path `fused_pipelined`
(ByteGrad and QAdam only) times the ByteGrad kernel's variant that sends the reduced chunks back
one destination at a time.

Bus bandwidth conventions (bytes that must cross each GPU's links, per direction):
  allreduce:  2(N-1)/N · S            bytegrad: 2(N-1)/N · (S/4 + 32N)
  shift_one:  S                        lp_ring:  2 · (S/4 + 32)
  allgather / alltoall / reduce_scatter: (N-1)/N · S      broadcast: S
Roofline fraction = busbw / 900 GB/s (nominal NVLink 5 per direction) and / 770 GB/s
(a measured peer-to-peer copy between two B200s through the NVSwitch).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bagua_core as bc  # noqa: E402
import bagua_core_b200 as bb  # noqa: E402
from bagua_core_b200.utils import flush_l2  # noqa: E402


def wire_bytes(op, S, N):
    if op in ("gradient_allreduce", "raw_nccl"):
        return 2 * (N - 1) / N * S
    if op in ("bytegrad", "qadam"):
        return 2 * (N - 1) / N * (S / 4 + 32 * N)
    if op == "shift_one":
        return S
    if op == "lp_ring":
        return 2 * (S / 4 + 32)
    if op in ("allgather", "alltoall", "reduce_scatter"):
        return (N - 1) / N * S
    if op == "broadcast":
        return S
    raise ValueError(op)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--ops", default="gradient_allreduce,bytegrad,shift_one,lp_ring,raw_nccl")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--paths", default="fused,library")
    ap.add_argument("--tunes", default="",
                    help="engine tuning sets to run the whole sweep under, separated by ';', each a comma-separated "
                         "list of key=value (bagua_core_b200._C.set_tuning), e.g. 'overlap_ctas=16;overlap_ctas=64'; "
                         "rows carry the set in `tune`")
    ap.add_argument("--comm-ctas", type=int, default=0, help="CTA budget of the all-reduce / pair kernels (0: default)")
    ap.add_argument("--coop-ctas", type=int, default=0, help="CTA budget of ByteGrad / ring kernels (0: default)")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    stream = torch.cuda.Stream(priority=-1)
    uid = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = bc.BaguaSingleCommunicatorPy(rank, world, local, stream.cuda_stream, uid[0])
    assert comm.fused_available()
    if args.comm_ctas or args.coop_ctas:
        comm.set_comm_ctas(args.comm_ctas, args.coop_ctas)
    backend = bc.BaguaCommBackendPy(100, local)
    defaults = dict(bb._C.get_tuning())

    sizes = []
    s = args.min_bytes
    while s <= args.max_bytes:
        sizes.append(s)
        s *= 4
    results = []
    align = 16 * world

    def time_bucket(bucket, tensor, iters, warmup):
        backend.register_ordered_buckets([bucket])

        def once():
            backend.mark_communication_ready(tensor, 0)

        for _ in range(warmup):
            once()
        backend.wait_pending_comm_ops()
        stream.synchronize()
        dist.barrier()
        flush_l2()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        for _ in range(iters):
            once()
        backend.wait_pending_comm_ops()
        with torch.cuda.stream(stream):
            e1.record()
        stream.synchronize()
        comm.check_device_status()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3  # µs

    tune_sets = [t for t in args.tunes.split(";") if t] or [""]
    for tune, op in [(t, o) for t in tune_sets for o in args.ops.split(",")]:
        for k, v in defaults.items():
            bb._C.set_tuning(k, int(v))
        for kv in [kv for kv in tune.split(",") if kv]:
            k, v = kv.split("=")
            bb._C.set_tuning(k, int(v))
        for S in sizes:
            n = max(align, (S // 4) // align * align)
            g = torch.Generator().manual_seed(rank)
            iters = args.iters if S <= (64 << 20) else max(3, args.iters // 4)
            for path in args.paths.split(","):
                if op == "raw_nccl" and path != "library":
                    continue
                if op == "shift_one" and world % 2:
                    continue
                # fused_pipelined: ByteGrad with the reduced chunks sent back one destination at a time
                # (the engine reads the variable at every call, so one process can time both variants)
                if path == "fused_pipelined":
                    if op not in ("bytegrad", "qadam"):
                        continue
                    os.environ["BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK"] = "0"
                else:
                    os.environ.pop("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", None)
                if path == "fused_sym":
                    # bucket in symmetric memory: peers load from and store into it directly, no staging
                    if op not in ("gradient_allreduce", "shift_one"):
                        continue
                    comm.set_fused(True)
                    x = comm.alloc_symmetric(n, torch.float32)
                    x.copy_(torch.randn(n, generator=g))
                else:
                    x = torch.randn(n, generator=g).to(dev)
                bt = bc.BaguaTensorPy(x, "x")
                bucket = bc.BaguaBucketPy(f"{op}_{S}", [bt])
                comm.set_fused(path != "library")
                bb._C.set_sync_per_bucket(path == "library")
                keep = []
                if op == "gradient_allreduce":
                    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True,
                                                             scattergather=False)
                elif op in ("bytegrad", "qadam"):
                    # QAdam's compression phase all-reduces the momentum buffer with the same compressed
                    # op that ByteGrad applies to gradients
                    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True,
                                                             scattergather=True, compression="MinMaxUInt8")
                elif op == "shift_one":
                    peer = torch.zeros_like(x)
                    keep.append(peer)
                    bucket.append_decentralized_synchronous_op(comm, None, hierarchical=False,
                                                               peer_selection_mode="shift_one",
                                                               peer_weight=bc.BaguaTensorPy(peer, "p"))
                elif op == "lp_ring":
                    w, l, r = x.clone(), x.clone(), x.clone()
                    keep += [w, l, r]
                    bucket.append_low_precision_decentralized_synchronous_op(
                        comm, None, hierarchical=False, peer_selection_mode="ring", compression="MinMaxUInt8",
                        weight=bc.BaguaTensorPy(w, "w"), left_peer_weight=bc.BaguaTensorPy(l, "l"),
                        right_peer_weight=bc.BaguaTensorPy(r, "r"))
                elif op == "raw_nccl":
                    comm.set_p2p_collectives(False)
                    bucket.append_python_op(lambda _name, bt=bt: comm.allreduce_inplace(bt, 10))
                elif op in ("allgather", "alltoall", "reduce_scatter", "broadcast"):
                    comm.set_p2p_collectives(path != "library")
                    part = torch.zeros(n // world, device=dev)
                    other = torch.zeros(n, device=dev)
                    keep += [part, other]
                    pt, ot = bc.BaguaTensorPy(part, "part"), bc.BaguaTensorPy(other, "other")
                    if op == "allgather":
                        bucket.append_python_op(lambda _name, a=pt, b=bt: comm.allgather(a, b))
                    elif op == "alltoall":
                        bucket.append_python_op(lambda _name, a=bt, b=ot: comm.alltoall(a, b))
                    elif op == "reduce_scatter":
                        bucket.append_python_op(lambda _name, a=bt, b=pt: comm.reduce_scatter(a, b, 10))
                    else:
                        bucket.append_python_op(lambda _name, b=bt: comm.broadcast(b, 0))
                us = time_bucket(bucket, bt, iters, args.warmup)
                wb = wire_bytes(op, n * 4, world)
                row = {"op": op, "path": path, "tune": tune, "bytes": n * 4, "n_gpus": world, "latency_us": us,
                       "busbw_gbs": wb / (us * 1e-6) / 1e9, "algbw_gbs": n * 4 / (us * 1e-6) / 1e9,
                       "frac_of_900": wb / (us * 1e-6) / 1e9 / 900.0, "frac_of_770_measured": wb / (us * 1e-6) / 1e9 / 770.0}
                results.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                del bucket, bt, x, keep
    bb._C.set_sync_per_bucket(False)
    comm.set_p2p_collectives(False)
    os.environ.pop("BAGUA_B200_BYTEGRAD_PIPELINE_MIN_CHUNK", None)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"n_gpus": world, "results": results, "stats": dict(bb._C.stats())}, f, indent=1)
    backend.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
