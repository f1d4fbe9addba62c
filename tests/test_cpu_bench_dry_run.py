"""bench.py end to end on CPU ranks (`--device cpu`: gloo, wall-clock timing, small MLP): the whole
benchmark logic — model build, `with_bagua`, device-timed loop, pipelined end-to-end loop, JSON line —
runs without a GPU, so mistakes in it are caught before it meets one.  The numbers mean nothing."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"}


def _line(out):
    lines = [ln for ln in out.splitlines() if ln.startswith("{") and '"metric"' in ln]
    assert len(lines) == 1, out[-3000:]
    return json.loads(lines[0])


def test_single_rank_dry_run_prints_one_contract_line():
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--device", "cpu", "--model", "mlp", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    line = _line(run.stdout)
    assert KEYS <= set(line)
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["value"] > 0
    assert line["e2e"]["loop"] == "pipelined" and line["e2e"]["value"] > 0 and line["e2e"]["h2d_bytes_per_step"] > 0
    assert line["gpu_launches"] > 0
    assert {"model", "global_batch", "parallelism"} <= set(line["config"])


def test_two_rank_dry_run_under_torchrun():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29633", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--device", "cpu", "--model", "mlp",
           "--steps", "2", "--warmup", "3"]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    line = _line(run.stdout)  # only rank 0 prints
    assert line["n_gpus"] == 2 and line["config"]["global_batch"] == 128 and line["config"]["parallelism"] == "dp2"


def test_reference_arm_reports_unavailable():
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True, text=True,
                         timeout=120, cwd=ROOT)
    assert run.returncode == 0
    rec = json.loads(run.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec
