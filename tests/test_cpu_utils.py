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
