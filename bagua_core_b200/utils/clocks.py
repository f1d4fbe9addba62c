"""Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs
(read-only queries; no GPU setting is ever changed)."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
import time
from typing import Dict, List

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Context manager around `nvidia-smi -lms`.  Call `mark()` right before the timed region
    starts (it first waits for the sampler's first line, so short regions still get samples);
    `summary()` then reports only samples taken after the mark.  Keep the period long and run one
    sampler per job, not one per rank: every query takes driver locks that kernel launches wait for."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc = None
        self._lines: List[str] = []
        self._thread = None
        self._mark = 0

    def __enter__(self):
        if shutil.which("nvidia-smi") is None:
            return self
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except Exception:
            self._proc = None
        return self

    def _read(self):
        for line in self._proc.stdout:
            self._lines.append(line.strip())

    def mark(self, wait_s: float = 3.0):
        """Wait (bounded) until the sampler has produced its first line, then start counting."""
        if self._proc is None:
            return
        deadline = time.time() + wait_s
        while not self._lines and time.time() < deadline:
            time.sleep(0.01)
        self._mark = len(self._lines)

    def __exit__(self, *exc):
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0 * 1.5)  # let the last sample of the region arrive
            self._proc.terminate()  # the exact child this object started
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
        return False

    def summary(self) -> Dict:
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self._lines[self._mark:] or self._lines[-3:]
        for line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                power.append(float(f[3]))
            except ValueError:
                pass
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}
