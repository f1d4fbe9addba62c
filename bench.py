#!/usr/bin/env python
"""Headline benchmark: training throughput (samples/s) of the named model/config through
the engine's public API (`with_bagua`), on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Default config: VGG-16 (138 M parameters), bf16 autocast with fp32 gradients, batch 32 per
GPU of 3x224x224 N(0,1) images, uniform labels over 1000 classes, gradient_allreduce with
10 MB buckets in reverse registration order, SGD momentum 0.9.  Other configs:
`--model bert_large --algorithm bytegrad`, `--model resnet50 --algorithm decentralized`.

`--impl` selects the arm: `ours` (fused sm_100a kernels), `baseline_nccl` (same engine,
library collectives replaying the reference's call sequence with a stream sync per
bucket), `ddp` (torch DistributedDataParallel), `reference` (the unmodified reference
package, which cannot be installed offline: prints an `unavailable` line).

Rank 0 prints ONE JSON line.  `value` is device-timed (CUDA events, barrier + synchronize
on both sides, max over ranks) with inputs resident on the device; `e2e.value` is the same
loop fed from pinned host memory every step and reading the loss back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline_nccl", "ddp"])
    ap.add_argument("--model", default="vgg16", choices=["vgg16", "bert_large", "resnet50", "mlp"])
    ap.add_argument("--algorithm", default=None,
                    choices=[None, "gradient_allreduce", "bytegrad", "decentralized", "decentralized_shift_one",
                             "low_precision_decentralized", "qadam", "async"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch size")
    ap.add_argument("--bucket-mb", type=float, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--repeats", type=int, default=5,
                    help="the timed block of --steps steps is run this many times; the line reports the median block "
                         "and lists all of them")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timed blocks, run a few more steps with two device events per bucket and report "
                         "how long each bucket's communication ran and how much of it was left after backward")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="engine tuning value (bagua_core_b200._C.set_tuning), e.g. overlap_ctas=16")
    ap.add_argument("--comm-ctas", type=int, default=0, help="CTA budget of the fused kernels (0: default)")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: dry run of the whole benchmark logic on host tensors (gloo, wall-clock timing); "
                         "its numbers are not benchmark results")
    ap.add_argument("--fused-model-ops", dest="fused_model_ops", action="store_true", default=None,
                    help="VGG-16: conv+bias+ReLU(+pool) blocks through this package's fused kernels "
                         "(the default for vgg16 on a GPU)")
    ap.add_argument("--no-fused-model-ops", dest="fused_model_ops", action="store_false",
                    help="VGG-16 built from plain Conv2d / ReLU / MaxPool2d modules")
    ap.add_argument("--bf16-shadow", action="store_true",
                    help="the optimizer kernel also writes bf16 copies of the weights and the fused blocks read those "
                         "instead of casting the fp32 master weights in every forward pass (same values; fused VGG-16 "
                         "and BERT, flat SGD optimizer; off by default until it has been timed)")
    ap.add_argument("--fused-wgrad", dest="fused_wgrad", action="store_true", default=None,
                    help="linear layers of the fused VGG-16 and of BERT add their weight gradient into the fp32 "
                         "gradient bucket with the GEMM that computes it, instead of a bf16 product, a cast and a "
                         "separate accumulation (the default for those models: 8 %% faster VGG-16 step on one B200)")
    ap.add_argument("--no-fused-wgrad", dest="fused_wgrad", action="store_false")
    return ap.parse_args()


CONFIGS = {
    # model: (default algorithm, per-GPU batch, bucket MB, seq_len)
    "vgg16": ("gradient_allreduce", 32, 10, None),
    "bert_large": ("bytegrad", 8, 25, 384),
    "resnet50": ("decentralized_shift_one", 128, 10, None),
    "mlp": ("gradient_allreduce", 64, 1, None),
}


def reference_arm(args):
    why = ("reference cannot be installed offline: pip metadata step fails with ModuleNotFoundError "
           "setuptools_rust; no cargo/rustc/mpicxx on the image, Aluminum submodule empty, installer downloads NCCL")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def build_model(name, device, fused_ops=False):
    import torch

    from bagua_core_b200 import models

    if name == "vgg16":
        m = models.VGG16(fused_ops=fused_ops).to(device).to(memory_format=torch.channels_last)
    elif name == "resnet50":
        m = models.ResNet50().to(device).to(memory_format=torch.channels_last)
    elif name == "bert_large":
        m = models.BertForQuestionAnswering(models.BertConfig.large()).to(device)
    else:
        m = models.MLP(1024, 4096, 1000, depth=4).to(device)
    return m


def make_batch(name, batch, seq, device, pinned=False):
    """Synthetic data of the benchmark's shape.  pinned=True → host tensors in pinned memory."""
    import torch

    g = torch.Generator().manual_seed(1 + int(os.environ.get("RANK", "0")))
    if name in ("vgg16", "resnet50"):
        x = torch.randn(batch, 3, 224, 224, generator=g)
        y = torch.randint(0, 1000, (batch,), generator=g)
    elif name == "bert_large":
        x = torch.randint(0, 30522, (batch, seq), generator=g)
        y = torch.randint(0, seq, (batch, 2), generator=g)
    else:
        x = torch.randn(batch, 1024, generator=g)
        y = torch.randint(0, 1000, (batch,), generator=g)
    if pinned:
        if device.type != "cuda":
            return x, y
        return x.pin_memory(), y.pin_memory()
    x = x.to(device)
    if x.dim() == 4:
        x = x.contiguous(memory_format=torch.channels_last)
    return x, y.to(device)


def loss_fn(name, model, x, y):
    import torch
    import torch.nn.functional as F

    import contextlib

    ctx = torch.autocast("cuda", dtype=torch.bfloat16) if x.is_cuda else contextlib.nullcontext()
    with ctx:
        if name == "bert_large":
            return model(x, y[:, 0], y[:, 1])
        out = model(x)
    return F.cross_entropy(out.float(), y)


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    import bagua_core_b200 as bb
    import bagua_core_b200.parallel as P
    from bagua_core_b200.utils import ClockSampler

    algo_name, batch, bucket_mb, seq = CONFIGS[args.model]
    algo_name = args.algorithm or algo_name
    batch = args.batch or batch
    bucket_mb = args.bucket_mb or bucket_mb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    on_gpu = args.device == "cuda"
    if on_gpu:
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        torch.backends.cudnn.benchmark = True
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    else:
        device = torch.device("cpu")
        if args.impl != "ours":
            raise SystemExit("--device cpu runs the default arm only")
    torch.manual_seed(0)

    class _Mark:
        """A point on the device's time line: a CUDA event, or the wall clock in a CPU dry run."""

        def __init__(self):
            self.ev = torch.cuda.Event(enable_timing=True) if on_gpu else None
            self.t = 0.0

        def record(self):
            if on_gpu:
                self.ev.record()
            else:
                self.t = time.perf_counter()

        def elapsed_time(self, other):
            return self.ev.elapsed_time(other.ev) if on_gpu else (other.t - self.t) * 1e3

    class _NoClocks:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

        def mark(self):
            pass

        def summary(self):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}

    if args.impl == "baseline_nccl":
        os.environ["BAGUA_B200_FUSED"] = "0"
        bb._C.set_sync_per_bucket(True)

    fused_ops = args.fused_model_ops
    if fused_ops is None:
        fused_ops = args.model == "vgg16" and on_gpu
    # the two linear-layer options need modules that honour them: the fused VGG-16 or BERT
    linear_opts = bool(fused_ops) or args.model == "bert_large"
    if args.fused_wgrad is None:
        args.fused_wgrad = linear_opts and on_gpu
    if args.impl == "ddp":
        args.fused_wgrad = False  # DDP's reducer does not learn of gradients through post-accumulate hooks
    if args.fused_wgrad and linear_opts:
        from bagua_core_b200.ops import wgrad

        wgrad.enabled = True
    model = build_model(args.model, device, fused_ops=fused_ops)
    if fused_ops and args.model == "vgg16":
        # One small forward/backward through the fused blocks before anything is timed; if it raises,
        # the benchmark runs the plain modules instead (same math, the framework's kernels).
        try:
            px, py_ = make_batch(args.model, 2, seq, device)
            loss_fn(args.model, model, px, py_).backward()
            for p in model.parameters():
                p.grad = None
            if on_gpu:
                torch.cuda.synchronize()
        except Exception as exc:
            print(f"[bench] fused model kernels failed ({exc!r}); using the plain modules", file=sys.stderr)
            fused_ops = False
            linear_opts = False  # the plain modules honour neither option
            torch.manual_seed(0)
            model = build_model(args.model, device, fused_ops=False)
    n_params = sum(p.numel() for p in model.parameters())
    lr = 0.01 if args.model != "bert_large" else 1e-4
    my_kernels = lambda: 0  # noqa: E731
    cpu_affinity = {}

    if args.impl == "ddp":
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9)
        fwd = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank],
                                                        bucket_cap_mb=bucket_mb, gradient_as_bucket_view=True)
        zero = lambda: opt.zero_grad(set_to_none=False)  # noqa: E731
    else:
        pg = P.init_process_group(device)
        cpu_affinity = dict(getattr(pg, "cpu_affinity", {}) or {})
        for kv in args.tune:
            k, v = kv.split("=")
            bb._C.set_tuning(k, int(v))
        if args.comm_ctas > 0 and on_gpu and world > 1:
            pg.global_comm.set_comm_ctas(args.comm_ctas, 0)
        if on_gpu and world > 1 and args.impl == "ours":
            _check_allreduce_paths(bb, pg, device, rank, world)
        if algo_name == "qadam":
            opt = P.QAdamOptimizer(model.parameters(), lr=1e-4, warmup_steps=2)
            algo = P.QAdamAlgorithm(opt)
        else:
            opt = P.FlatSGD(model.parameters(), lr=lr, momentum=0.9, bf16_shadow=bool(args.bf16_shadow and linear_opts))
            algo = {
                "gradient_allreduce": lambda: P.GradientAllReduceAlgorithm(),
                "bytegrad": lambda: P.ByteGradAlgorithm(),
                "decentralized": lambda: P.DecentralizedAlgorithm(peer_selection_mode="all"),
                "decentralized_shift_one": lambda: P.DecentralizedAlgorithm(
                    peer_selection_mode="shift_one" if world % 2 == 0 else "all"),
                "low_precision_decentralized": lambda: P.LowPrecisionDecentralizedAlgorithm(),
                "async": lambda: P.AsyncModelAverageAlgorithm(sync_interval_ms=50),
            }[algo_name]()
        fwd = P.with_bagua(model, [opt], algo, bucket_bytes=int(bucket_mb * 1024 * 1024))
        zero = lambda: opt.zero_grad(set_to_none=False)  # noqa: E731

        def my_kernels():
            s = bb._C.stats()
            from bagua_core_b200.ops import fused_conv

            return int(s["fused_launches"]) + int(getattr(opt, "kernel_launches", 0)) + fused_conv.launches

    def step(x, y):
        zero()
        loss = loss_fn(args.model, fwd, x, y)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    # ---- device-timed loop, inputs resident on the device -----------------------------
    # The block of `steps` steps is timed `repeats` times, each time bracketed by a barrier and a
    # synchronize on both sides and reduced to the maximum over ranks; the line reports the median
    # block, so that one hiccup in a region of a tenth of a second does not decide the number.
    x, y = make_batch(args.model, batch, seq, device)
    for _ in range(max(args.warmup, 3)):
        step(x, y)
    # The model, the optimizer and the engine's objects are long-lived: take them out of the garbage
    # collector's generations, so that a full collection on one rank does not land in a timed block
    # (every rank waits for the slowest one at each bucket).  Collection itself stays on.
    import gc

    gc.collect()
    gc.freeze()
    barrier()
    block_ms, block_launches = [], []
    # One sampler for the job (rank 0's GPU, every 100 ms): every NVML query takes driver locks that
    # kernel launches of all ranks wait for, and one `nvidia-smi -lms 50` per rank (160 query rounds
    # a second with eight ranks) showed up in the step time.
    with (ClockSampler(local_rank, period_ms=100) if on_gpu and rank == 0 else _NoClocks()) as clocks:
        clocks.mark()
        for _ in range(max(1, args.repeats)):
            k0 = my_kernels()
            e0, e1 = _Mark(), _Mark()
            barrier()
            e0.record()
            for _ in range(args.steps):
                step(x, y)
            e1.record()
            barrier()
            block_ms.append(e0.elapsed_time(e1))
            block_launches.append(my_kernels() - k0)
    t = torch.tensor(block_ms, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    block_ms = [float(v) for v in t.tolist()]
    order = sorted(range(len(block_ms)), key=lambda i: block_ms[i])
    pick = order[len(order) // 2]
    ms = block_ms[pick]
    launches = block_launches[pick]
    value = world * batch * args.steps / (ms / 1e3)

    # How long the launching thread needs to ISSUE one step (queue empty, nothing to wait for): when this
    # approaches ms_per_step the loop is bound by the host, not by the GPU.
    host_issue = []
    for _ in range(5):
        barrier()
        t_h = time.perf_counter()
        step(x, y)
        host_issue.append((time.perf_counter() - t_h) * 1e3)
    barrier()
    host_issue.sort()
    host_issue_ms = host_issue[len(host_issue) // 2]

    # ---- optional: device time line of the buckets' communication ------------------------
    timeline = None
    if args.timeline and on_gpu and args.impl != "ddp":
        timeline = bucket_timeline(bb, step, x, y, barrier, steps=4)

    # ---- end to end: pinned host inputs in, loss out, every step -----------------------
    e2e = None
    if not args.no_e2e:
        hx, hy = make_batch(args.model, batch, seq, device, pinned=True)
        h2d = hx.numel() * hx.element_size() + hy.numel() * hy.element_size()

        def e2e_step():
            dx = hx.to(device, non_blocking=True)
            if dx.dim() == 4 and on_gpu:
                dx = dx.contiguous(memory_format=torch.channels_last)
            dy = hy.to(device, non_blocking=True)
            return float(step(dx, dy).item())  # 4-byte device→host read of the loss

        def e2e_loop_plain(n):
            last = None
            for _ in range(n):
                last = e2e_step()
            return last

        def e2e_loop_pipelined(n):
            """Same work per step (one host→device copy of the batch, one device→host read of a loss), but
            the copy of batch k+1 runs on a side stream under step k and the loss of step k is read while
            the next three steps are already queued (a host that runs only one step ahead idles the GPU at
            every hiccup); all n losses are read before the function returns."""
            from bagua_core_b200.utils.prefetch import DevicePrefetcher, LaggedScalarReader

            pf, reader = DevicePrefetcher(device), LaggedScalarReader(device, lag=3)
            pf.put(hx, hy)
            for i in range(n):
                dx, dy = pf.get()
                if i + 1 < n:
                    pf.put(hx, hy)
                reader.push(step(dx, dy))
            return reader.flush()

        e2e_loop, e2e_mode = e2e_loop_pipelined, "pipelined"
        if os.environ.get("BAGUA_B200_BENCH_E2E", "pipelined") == "plain":
            e2e_loop, e2e_mode = e2e_loop_plain, "plain"
        failed = 0
        try:
            e2e_loop(3)
        except Exception as exc:  # the plain loop is the known-good fallback
            print(f"[bench] pipelined end-to-end loop failed ({exc!r}); using the plain loop", file=sys.stderr)
            failed = 1
        if world > 1:
            # Every rank takes the same loop: a rank that fell back alone would run three more
            # warm-up steps than its peers, and their collectives would no longer pair up.
            f = torch.tensor([failed], device=device, dtype=torch.int32)
            dist.all_reduce(f, op=dist.ReduceOp.MAX)
            failed = int(f.item())
        if failed and e2e_mode != "plain":
            e2e_loop, e2e_mode = e2e_loop_plain, "plain"
            e2e_loop(3)
        e2e_ms = []
        for _ in range(max(1, args.repeats)):
            e0, e1 = _Mark(), _Mark()
            barrier()
            e0.record()
            t0 = time.perf_counter()
            last = e2e_loop(args.steps)
            e1.record()
            barrier()
            wall_ms = (time.perf_counter() - t0) * 1e3
            e2e_ms.append(max(e0.elapsed_time(e1), wall_ms))  # the host read makes both agree; keep the slower
        t = torch.tensor(e2e_ms, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = sorted(float(v) for v in t.tolist())
        ems = e2e_ms[len(e2e_ms) // 2]
        e2e = {"value": world * batch * args.steps / (ems / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "ms_per_step": ems / args.steps,
               "last_loss": last, "loop": e2e_mode,
               "timed_blocks": {"n": len(e2e_ms), "reported": "median", "ms_per_step": [m / args.steps for m in e2e_ms]}}

    if rank == 0:
        line = {
            "metric": f"{args.model} training throughput ({algo_name})",
            "value": value,
            "unit": "samples/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16" if on_gpu else "fp32 (cpu dry run)",
            "data": "synthetic (N(0,1) inputs, uniform labels), random-init weights",
            "impl": args.impl,
            "config": {
                "model": args.model, "params": n_params, "global_batch": world * batch, "seq_len": seq,
                "parallelism": f"dp{world}", "algorithm": algo_name, "bucket_mb": bucket_mb,
                "optimizer": "sgd momentum 0.9" if algo_name != "qadam" else "qadam",
                "precision": "bf16 autocast, fp32 master weights and gradients",
                "fused_model_ops": bool(fused_ops),
                "bf16_weight_copies": bool(args.bf16_shadow and linear_opts and args.impl != "ddp" and algo_name != "qadam"),
                "fused_wgrad": _wgrad_report(args, linear_opts),
                "l2": "working set per step (fp32 weights+grads+momentum and activations) exceeds the 126 MB L2",
            },
            "clocks": clocks.summary(),
            "e2e": e2e,
            "gpu_launches": launches,
            "timed_blocks": {"n": len(block_ms), "reported": "median", "ms_per_step": [m / args.steps for m in block_ms]},
            "host_issue_ms_per_step": host_issue_ms,
            "cpu_affinity": cpu_affinity,
        }
        if timeline is not None:
            line["bucket_timeline"] = timeline
        print(json.dumps(line))
    if args.impl != "ddp":
        if hasattr(algo, "abort"):
            algo.abort(fwd)  # stop the background averaging thread before tearing down
        P.destroy_process_group()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


def _check_allreduce_paths(bb, pg, device, rank, world):
    """Before anything is timed: one 16 MB all-reduce through the copy-engine path and one through the
    bulk-copy kernel, checked against the known answer.  A path that gives a wrong result on this machine is
    switched off on every rank (the load/store kernels then serve its sizes) and the fact is printed."""
    import torch
    import torch.distributed as dist

    from bagua_core_b200 import BaguaTensorPy

    comm = pg.global_comm
    if not comm.fused_available():
        return
    n = 4 << 20
    buf = comm.alloc_symmetric(n, torch.float32)
    if buf is None:
        return
    want = (world + 1) / 2.0
    bt = BaguaTensorPy(buf, "bench_path_check")
    before = dict(bb._C.get_tuning())
    bad = {"ce_min_bytes": 0, "tma_min_bytes": 0}
    for key in bad:
        buf.fill_(float(rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        try:
            if key == "ce_min_bytes":
                ok = comm.fused_allreduce_ce(bt, bt, True)
            else:
                bb._C.set_tuning("tma_min_bytes", 1 << 20)
                bb._C.set_tuning("tma_isolated", 1)
                ok = comm.fused_allreduce(bt, bt, True) if world in (2, 4, 8) else True
            pg.comm_stream.synchronize()
            if ok and not bool(torch.all(buf == want).item()) and (key == "ce_min_bytes" or world in (2, 4, 8)):
                bad[key] = 1
        finally:
            bb._C.set_tuning("tma_min_bytes", before["tma_min_bytes"])
            bb._C.set_tuning("tma_isolated", before["tma_isolated"])
    flags = torch.tensor([bad["ce_min_bytes"], bad["tma_min_bytes"]], device=device, dtype=torch.int32)
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    for key, flag in zip(("ce_min_bytes", "tma_min_bytes"), flags.tolist()):
        if flag:
            bb._C.set_tuning(key, -1)
            if rank == 0:
                print(f"[bench] the all-reduce path behind `{key}` gave a wrong result in the start-up check; "
                      "switched off", file=sys.stderr)


def bucket_timeline(bb, step, x, y, barrier, steps=4):
    """Runs `steps` more steps with the engine's device time line on and returns, per step (mean over the
    steps): when backward ended, when the last bucket's communication ended, the communication left exposed
    after backward, and each bucket's start/end relative to the start of the step (all in ms, this rank)."""
    bb._C.timeline_collect()
    bb._C.set_bucket_timing(True)
    try:
        barrier()
        for _ in range(steps):
            step(x, y)
        barrier()
    finally:
        bb._C.set_bucket_timing(False)
    spans = bb._C.timeline_collect()
    per_step, cur = [], None
    for sp in spans:
        if sp["kind"] == "mark" and sp["name"] == "step_begin":
            cur = {"t0": sp["start_ms"], "backward_end": None, "buckets": []}
            per_step.append(cur)
        elif cur is None:
            continue
        elif sp["kind"] == "mark" and sp["name"] == "backward_end":
            cur["backward_end"] = sp["start_ms"] - cur["t0"]
        elif sp["kind"] == "bucket":
            cur["buckets"].append((sp["name"], sp["start_ms"] - cur["t0"], sp["end_ms"] - cur["t0"], sp["bytes"]))
    per_step = [s for s in per_step if s["backward_end"] is not None and s["buckets"]]
    if not per_step:
        return {"steps": 0}
    n = len(per_step)
    names = [b[0] for b in per_step[0]["buckets"]]
    buckets = []
    for i, name in enumerate(names):
        rows = [s["buckets"][i] for s in per_step if len(s["buckets"]) == len(names)]
        if not rows:
            continue
        buckets.append({"name": name, "mb": round(rows[0][3] / 2 ** 20, 2),
                        "start_ms": round(sum(r[1] for r in rows) / len(rows), 3),
                        "end_ms": round(sum(r[2] for r in rows) / len(rows), 3),
                        "busy_ms": round(sum(r[2] - r[1] for r in rows) / len(rows), 3)})
    bwd = sum(s["backward_end"] for s in per_step) / n
    last = sum(max(b[2] for b in s["buckets"]) for s in per_step) / n
    exposed = sum(max(0.0, max(b[2] for b in s["buckets"]) - s["backward_end"]) for s in per_step) / n
    return {"steps": n, "backward_end_ms": round(bwd, 3), "last_bucket_end_ms": round(last, 3),
            "exposed_comm_ms": round(exposed, 3), "comm_busy_ms": round(sum(b["busy_ms"] for b in buckets), 3),
            "buckets": buckets}


def _wgrad_report(args, linear_opts):
    """False, or which library call accumulated the weight gradients and how often it did / declined."""
    if not (args.fused_wgrad and linear_opts):
        return False
    from bagua_core_b200.ops import wgrad

    return {"mode": wgrad.cuda_mode or "host", "accumulated": wgrad.accumulated, "declined": wgrad.declined}


if __name__ == "__main__":
    sys.exit(main())
