#!/usr/bin/env python
"""What does a communication kernel of a given shape cost the backward pass it overlaps?

    python benchmarks/interference_probe.py [--steps 20] [--configs "64,512,2.5,0;16,512,2.5,0;..."]

Runs `bench.py` on ONE GPU several times.  With one rank a gradient bucket has nothing to
communicate; `BAGUA_B200_PROBE_OCCUPY=ctas,threads,us_per_mb,mode` makes the engine launch a
stand-in kernel in the bucket's place instead: on the communication stream, at the moment the
bucket becomes ready, resident for 15 us + us_per_mb per MB of the bucket.  mode 0 only
occupies its blocks (no memory traffic), mode 1 also streams over the bucket.  The step time
against the run without a stand-in is what a communication kernel of that grid, block size and
duration takes away from the compute kernels — separately for SM occupancy and for memory
traffic, and without a second GPU.  Prints one line per configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DEFAULT = ";".join([
    "64,512,2.5,0", "64,512,2.5,1", "16,512,2.5,0", "16,512,6,0", "128,128,2.5,0", "256,128,2.5,0", "148,64,2.5,0",
    "32,1024,2.5,0", "64,512,1.3,0",
])


def run(env_value, steps, model):
    env = dict(os.environ)
    if env_value:
        env["BAGUA_B200_PROBE_OCCUPY"] = env_value
    else:
        env.pop("BAGUA_B200_PROBE_OCCUPY", None)
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "1", "--steps", str(steps), "--warmup", "5",
           "--no-e2e", "--repeats", "3", "--timeline", "--model", model]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    if out.returncode != 0:
        return None, out.stderr[-800:]
    return json.loads(out.stdout.strip().splitlines()[-1]), ""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--model", default="vgg16")
    ap.add_argument("--configs", default=DEFAULT, help="';'-separated ctas,threads,us_per_mb,mode")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rows = []
    for cfg in [""] + [c for c in args.configs.split(";") if c]:
        d, err = run(cfg, args.steps, args.model)
        if d is None:
            print(json.dumps({"config": cfg, "error": err}), flush=True)
            continue
        t = d.get("bucket_timeline") or {}
        row = {"config": cfg or "none", "ms_per_step": round(d["ms_per_step"], 3),
               "backward_end_ms": t.get("backward_end_ms"), "standin_busy_ms": t.get("comm_busy_ms"),
               "exposed_ms": t.get("exposed_comm_ms")}
        if rows:
            row["cost_ms"] = round(row["ms_per_step"] - rows[0]["ms_per_step"], 3)
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
