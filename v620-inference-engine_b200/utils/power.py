"""GPU power integrated over a timed region, read-only, through NVML (``pynvml``): a thread samples every device's
power draw, ``stop()`` returns seconds, average watts and kilojoules.  The prefix cache is justified by energy (a
recompute runs the GPUs at full power for seconds), so the cache benches report joules next to seconds.  GPUs only;
the sensor's own averaging window is about a second, so short regions read coarsely.
(Role of the reference's bench/power_meter.hpp, which integrates the cards' hwmon sensors.)"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional


def nvml_reader(indices: Optional[List[int]] = None) -> Optional[Callable[[], float]]:
    """A function returning the summed power draw in watts, or None when NVML is not available."""
    try:
        import pynvml
        pynvml.nvmlInit()
        n = pynvml.nvmlDeviceGetCount()
        hs = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in (indices if indices is not None else range(n))]
        return lambda: sum(pynvml.nvmlDeviceGetPowerUsage(h) for h in hs) / 1000.0
    except Exception:
        return None


class PowerMeter:
    def __init__(self, read_watts: Optional[Callable[[], float]] = None, period_s: float = 0.05, indices: Optional[List[int]] = None):
        self.read = read_watts if read_watts is not None else nvml_reader(indices)
        self.period = period_s
        self._stop = threading.Event()
        self._th: Optional[threading.Thread] = None
        self.joules = 0.0
        self.t0 = self.t1 = 0.0

    def _run(self):
        # the integral covers exactly [t0, t1]: the first reading stands for the moment of start() (the thread may come up a
        # little later), the last one for the moment of stop()
        last_t, last_w = self.t0, self.read()
        while not self._stop.wait(self.period):
            t, w = time.perf_counter(), self.read()
            self.joules += 0.5 * (w + last_w) * (t - last_t)          # trapezoid between two samples
            last_t, last_w = t, w
        w = self.read()
        self.joules += 0.5 * (w + last_w) * max(0.0, self.t1 - last_t)

    def start(self) -> "PowerMeter":
        self.joules = 0.0
        self._stop.clear()
        self.t0 = time.perf_counter()
        if self.read is not None:
            self._th = threading.Thread(target=self._run, daemon=True)
            self._th.start()
        return self

    def stop(self) -> dict:
        self.t1 = time.perf_counter()
        self._stop.set()
        if self._th is not None:
            self._th.join()
            self._th = None
        s = self.t1 - self.t0
        if self.read is None:
            return {"seconds": round(s, 4), "ok": False}
        return {"seconds": round(s, 4), "avg_w": round(self.joules / max(s, 1e-9), 1), "kilojoules": round(self.joules / 1e3, 4), "ok": True}
