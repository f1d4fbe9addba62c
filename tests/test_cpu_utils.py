"""Measurement helpers, exercised without a GPU (a stand-in `nvidia-smi` on PATH)."""
import os
import stat
import time

from bagua_core_b200.utils import ClockSampler, load_measured_peaks

FAKE = """#!/bin/sh
# prints one CSV line per 20 ms, like `nvidia-smi --query-gpu=... -lms 20`
i=0
while [ $i -lt 200 ]; do
  if [ $i -lt 5 ]; then
    echo "0, 345, 1965, 180.5, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active"
  else
    echo "0, 1320, 1965, 998.2, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
  fi
  i=$((i+1))
  sleep 0.02
done
"""


def test_clock_sampler_reports_only_the_marked_region(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    with ClockSampler(0, period_ms=20) as c:
        time.sleep(0.3)  # idle samples (345 MHz) arrive before the mark
        c.mark()
        time.sleep(0.3)
    s = c.summary()
    assert s["samples"] >= 5
    assert s["sm_mhz"] == 1320.0 and s["sm_max_mhz"] == 1965.0
    assert s["reasons"] == ["sw_power_cap"]
    assert s["power_w_max"] > 900


def test_clock_sampler_without_nvidia_smi(monkeypatch, tmp_path):
    monkeypatch.setenv("PATH", str(tmp_path))
    with ClockSampler(0) as c:
        c.mark()
    assert c.summary()["samples"] == 0


def test_measured_peaks_have_the_fields_the_benchmarks_use():
    p = load_measured_peaks()
    assert p["hbm_gbs"] > 1000 and p["bf16_tflops"] > 100 and p["source"] in ("measured", "fallback")


def test_conv_bias_relu_module_is_a_drop_in_on_cpu():
    """Off the fused path (CPU, fp32) the module is exactly Conv2d followed by ReLU, with Conv2d's state dict."""
    import torch

    from bagua_core_b200.models import VGG16
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU

    torch.manual_seed(0)
    fused = ConvBiasReLU(3, 8, 3, padding=1)
    plain = torch.nn.Conv2d(3, 8, 3, padding=1)
    plain.load_state_dict(fused.state_dict())
    x = torch.randn(2, 3, 9, 9, requires_grad=True)
    y = fused(x)
    assert torch.equal(y, torch.relu(plain(x)))
    y.sum().backward()
    assert fused.bias.grad is not None and x.grad is not None
    a, b = VGG16(num_classes=10, fused_ops=True), VGG16(num_classes=10)
    assert sum(p.numel() for p in a.parameters()) == sum(p.numel() for p in b.parameters())
    assert [tuple(p.shape) for p in a.parameters()] == [tuple(p.shape) for p in b.parameters()]


def test_prefetcher_and_lagged_reader_on_cpu():
    """On a CPU device the pipelining helpers are plain pass-throughs with the same call pattern."""
    import torch

    from bagua_core_b200.utils.prefetch import DevicePrefetcher, LaggedScalarReader

    pf, reader = DevicePrefetcher(torch.device("cpu")), LaggedScalarReader(torch.device("cpu"))
    seen = []
    pf.put(torch.tensor([1.0]), torch.tensor([2]))
    for i in range(3):
        x, y = pf.get()
        pf.put(torch.tensor([float(i + 2)]), torch.tensor([i]))
        seen.append(reader.push(x.sum()))
    assert seen == [None, 1.0, 2.0]
    assert reader.flush() == 3.0 and reader.flush() is None
    import pytest

    pf.get()
    with pytest.raises(RuntimeError):
        pf.get()


def test_lagged_reader_with_a_deeper_lag_returns_every_value_once_and_in_order():
    import torch

    from bagua_core_b200.utils.prefetch import LaggedScalarReader

    reader = LaggedScalarReader(torch.device("cpu"), lag=3)
    got = [reader.push(torch.tensor(float(i))) for i in range(6)]
    assert got == [None, None, None, 0.0, 1.0, 2.0]
    assert reader.flush() == 5.0  # 3.0 and 4.0 were read on the way
    assert reader.flush() is None


class _FakeNvml:
    """Stands for the NVML binding: one GPU whose local CPUs are `cpus`."""

    def __init__(self, cpus, fail=False, gpus=1):
        self.cpus, self.fail, self.calls, self.gpus = set(cpus), fail, [], gpus

    def nvmlDeviceGetCount(self):
        return self.gpus

    def nvmlInit(self):
        if self.fail:
            raise RuntimeError("no driver")
        self.calls.append("init")

    def nvmlShutdown(self):
        self.calls.append("shutdown")

    def nvmlDeviceGetHandleByUUID(self, uuid):
        self.calls.append(("uuid", uuid))
        if isinstance(uuid, bytes):
            raise TypeError("str expected")
        return "h"

    def nvmlDeviceGetHandleByIndex(self, i):
        self.calls.append(("index", i))
        return "h"

    def nvmlDeviceGetCpuAffinity(self, handle, n_words):
        words = [0] * n_words
        for c in self.cpus:
            if c // 64 < n_words:
                words[c // 64] |= 1 << (c % 64)
        return words


def test_cpu_affinity_follows_the_gpus_local_cpus_and_only_narrows(monkeypatch):
    import os
    import threading

    from bagua_core_b200.utils import affinity

    assert affinity._mask_words_to_cpus([0b101, 1]) == {0, 2, 64}
    before = set(os.sched_getaffinity(0))
    if len(before) < 4:
        pytest.skip("needs four CPUs")
    half = set(sorted(before)[: len(before) // 2])
    stop = threading.Event()
    seen = {}

    def other_thread():
        stop.wait()
        seen["mask"] = set(os.sched_getaffinity(0))

    th = threading.Thread(target=other_thread)
    th.start()
    try:
        monkeypatch.delenv("BAGUA_B200_CPU_AFFINITY", raising=False)
        # too few of the GPU's CPUs are ours: nothing changes
        r = affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=_FakeNvml({max(before) + 1000, min(before)}))
        assert r["applied"] is False and set(os.sched_getaffinity(0)) == before
        # NVML not there: nothing changes
        r = affinity.bind_to_gpu_cpus(0, nvml=_FakeNvml(half, fail=True))
        assert r["applied"] is False and set(os.sched_getaffinity(0)) == before
        # switched off
        monkeypatch.setenv("BAGUA_B200_CPU_AFFINITY", "0")
        assert affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=_FakeNvml(half))["reason"] == "switched off"
        monkeypatch.delenv("BAGUA_B200_CPU_AFFINITY")
        # the GPU's CPUs, cut to what the process may use; found by UUID; every thread moves
        fake = _FakeNvml(half | {max(before) + 1000})
        r = affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=fake, uuid="1234")
        assert r == {"applied": True, "cpus": len(half), "reason": ""}
        assert ("uuid", "GPU-1234") in fake.calls and fake.calls[-1] == "shutdown"
        assert set(os.sched_getaffinity(0)) == half
        stop.set()
        th.join()
        assert seen["mask"] == half
        # eight GPUs report the same few CPUs: binding eight ranks there would crowd them, so it is refused
        for tid in affinity._all_thread_ids():
            try:
                os.sched_setaffinity(tid, before)
            except OSError:
                pass  # a thread of an earlier test that has just exited
        r = affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=_FakeNvml(half, gpus=8), per_rank_cpus=len(half))
        assert r["applied"] is False and "8 GPU(s) share" in r["reason"] and set(os.sched_getaffinity(0)) == before
        assert affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=_FakeNvml(half))["applied"] is True
        # a second call finds nothing to do
        assert affinity.bind_to_gpu_cpus(0, min_cpus=2, nvml=_FakeNvml(half))["reason"] == "already there"
    finally:
        stop.set()
        th.join()
        for tid in affinity._all_thread_ids():
            try:
                os.sched_setaffinity(tid, before)
            except OSError:
                pass
