"""Sample GPU clocks and throttle reasons with ``nvidia-smi`` while a timed region runs.

Read-only: nothing here changes a GPU setting.  ``ClockSampler`` starts ``nvidia-smi -lms`` as a
child process writing CSV to a file, and ``summary()`` reduces the samples taken under load to
the median SM clock, the maximum clock and the set of throttle reasons that were active.
"""
from __future__ import annotations

import os
import signal
import statistics
import subprocess
import tempfile
import time
from typing import Dict, List, Optional

FIELDS = ["index", "clocks.sm", "clocks.max.sm", "power.draw", "clocks_event_reasons.active",
          "clocks_event_reasons.hw_slowdown", "clocks_event_reasons.hw_thermal_slowdown",
          "clocks_event_reasons.sw_thermal_slowdown", "clocks_event_reasons.sw_power_cap"]


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu, self.period = gpu_index, period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.path = os.path.join(tempfile.gettempdir(), f"qw_clocks_{os.getpid()}_{gpu_index}.csv")
        self.t0 = self.t1 = 0.0

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={','.join(FIELDS)}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", str(self.period)], stdout=self.f, stderr=subprocess.DEVNULL)
        except (OSError, FileNotFoundError):
            self.proc = None
        self.t0 = time.time()

    def stop(self):
        self.t1 = time.time()
        if self.proc is not None:
            try:
                self.proc.send_signal(signal.SIGTERM)     # the exact child we started
                self.proc.wait(timeout=5)
            except Exception:
                pass
            self.f.close()

    def summary(self) -> Dict[str, object]:
        rows: List[List[str]] = []
        try:
            with open(self.path) as f:
                rows = [[c.strip() for c in ln.split(",")] for ln in f if ln.strip()]
        except OSError:
            pass
        sm, mx, reasons, power = [], [], set(), []
        for r in rows:
            if len(r) < len(FIELDS):
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "under load": samples at or above the median power draw
        cut = statistics.median(power)
        load = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}
