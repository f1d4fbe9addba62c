#!/usr/bin/env python
"""Minimal training script: any benchmark model with any algorithm on synthetic data.

    python examples/train_synthetic.py --model mlp --algorithm gradient_allreduce --steps 20
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_synthetic.py \
        --model vgg16 --algorithm bytegrad

Runs on CPU ranks (gloo) when no GPU is visible.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bagua_core_b200.parallel as P  # noqa: E402
from bagua_core_b200 import models  # noqa: E402
from bagua_core_b200.utils import DevicePrefetcher, LaggedScalarReader  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mlp", choices=["mlp", "vgg16", "resnet50"])
    ap.add_argument("--algorithm", default="gradient_allreduce",
                    choices=["gradient_allreduce", "bytegrad", "decentralized", "shift_one", "low_precision", "qadam",
                             "async"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8)
    args = ap.parse_args()

    pg = P.init_process_group()
    dev = pg.device
    torch.manual_seed(0)
    if args.model == "mlp":
        model, shape, classes = models.MLP(64, 256, 10), (64,), 10
    elif args.model == "vgg16":
        model, shape, classes = models.VGG16(), (3, 224, 224), 1000
    else:
        model, shape, classes = models.ResNet50(), (3, 224, 224), 1000
    model = model.to(dev)
    if args.algorithm == "qadam":
        opt = P.QAdamOptimizer(model.parameters(), lr=1e-3, warmup_steps=max(1, args.steps // 2))
        algo = P.QAdamAlgorithm(opt)
    else:
        opt = P.FlatSGD(model.parameters(), lr=0.01, momentum=0.9)
        algo = {
            "gradient_allreduce": P.GradientAllReduceAlgorithm,
            "bytegrad": P.ByteGradAlgorithm,
            "decentralized": lambda: P.DecentralizedAlgorithm(peer_selection_mode="all"),
            "shift_one": lambda: P.DecentralizedAlgorithm(
                peer_selection_mode="shift_one" if pg.world_size % 2 == 0 else "all"),
            "low_precision": P.LowPrecisionDecentralizedAlgorithm,
            "async": lambda: P.AsyncModelAverageAlgorithm(sync_interval_ms=100),
        }[args.algorithm]()
    model = P.with_bagua(model, [opt], algo)
    g = torch.Generator().manual_seed(pg.rank)

    def host_batch():
        x = torch.randn(args.batch, *shape, generator=g)
        y = torch.randint(0, classes, (args.batch,), generator=g)
        return (x.pin_memory(), y.pin_memory()) if dev.type == "cuda" else (x, y)

    # the next batch is copied on a side stream while this step computes; each loss is read one step
    # late, so the launch thread never waits for the GPU
    prefetch, losses = DevicePrefetcher(dev, channels_last=False), LaggedScalarReader(dev)
    prefetch.put(*host_batch())
    for step in range(args.steps):
        x, y = prefetch.get()
        if step + 1 < args.steps:
            prefetch.put(*host_batch())
        opt.zero_grad(set_to_none=False)
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        previous = losses.push(loss)
        if pg.rank == 0 and previous is not None:
            print(f"step {step - 1}: loss {previous:.4f}")
    if pg.rank == 0:
        print(f"step {args.steps - 1}: loss {losses.flush():.4f}")
    if hasattr(algo, "abort"):
        algo.abort(model)
    P.destroy_process_group()


if __name__ == "__main__":
    main()
