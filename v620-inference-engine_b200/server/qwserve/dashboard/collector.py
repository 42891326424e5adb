"""Samples the scheduler's counters and, where NVML is present, each GPU's utilisation, memory, power, temperature
and SM clock once a second (reference behaviour: server/qwserve/dashboard/collector.py:12-95).  NVML is only
read, never written."""
import threading
import time

from .metrics import Metrics


class Gpus:
    """Read-only NVML view; ``nvml`` may be a stand-in object with the same functions (tests)."""

    def __init__(self, nvml=None):
        self.nv, self.handles = None, []
        try:
            if nvml is None:
                import pynvml as nvml
            nvml.nvmlInit()
            self.nv = nvml
            self.handles = [nvml.nvmlDeviceGetHandleByIndex(i) for i in range(nvml.nvmlDeviceGetCount())]
        except Exception:
            self.nv = None

    def sample(self) -> list:
        out = []
        nv = self.nv
        for i, h in enumerate(self.handles):
            try:
                u = nv.nvmlDeviceGetUtilizationRates(h)
                m = nv.nvmlDeviceGetMemoryInfo(h)
                out.append({"index": i, "util": float(u.gpu), "mem_used_gb": m.used / 2**30, "mem_total_gb": m.total / 2**30,
                            "power_w": nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                            "temp_c": float(nv.nvmlDeviceGetTemperature(h, 0)),
                            "sm_mhz": float(nv.nvmlDeviceGetClockInfo(h, 1))})
            except Exception:
                out.append({"index": i})
        return out


class Collector:
    def __init__(self, server, nvml=None, period: float = 1.0):
        self.server, self.period = server, period
        self.metrics = Metrics()
        self.gpus = Gpus(nvml)
        self.gpu_last: list = []
        self.stop_flag = threading.Event()
        self.thread = threading.Thread(target=self._run, name="qw-metrics", daemon=True)

    def start(self):
        self.thread.start()

    def stop(self):
        self.stop_flag.set()

    def sample_once(self, now: float = None) -> dict:
        now = now if now is not None else time.time()
        c = self.server.sched.counts()
        cs = self.server.sched.cache_stats or {}
        s = {"tok_s": self.metrics.rate("tokens", c.get("tokens", 0), now), "req_s": self.metrics.rate("completed", c.get("completed", 0), now),
             "waiting": c.get("waiting", 0), "prefilling": c.get("prefilling", 0), "running": c.get("running", 0),
             "step_ms": c.get("step_ms", 0.0), "failed": c.get("failed", 0),
             "cache_reused_tokens": cs.get("reused_tokens", 0), "cache_ram_gb": cs.get("ram_bytes", 0) / 2**30,
             "cache_disk_gb": cs.get("disk_bytes", 0) / 2**30}
        self.gpu_last = self.gpus.sample()
        for g in self.gpu_last:
            for k in ("util", "power_w", "mem_used_gb"):
                if k in g:
                    s[f"gpu{g['index']}_{k}"] = g[k]
        self.metrics.push(s, now)
        return s

    def _run(self):
        while not self.stop_flag.wait(self.period):
            try:
                self.sample_once()
            except Exception:
                pass

    def payload(self, tail: int = 300) -> dict:
        reason = self.server.sched.health()
        return {"model": self.server.model_name, "healthy": reason is None, "reason": reason, "gpus": self.gpu_last,
                "counts": self.server.sched.counts(), "prefix_cache": self.server.sched.cache_stats, **self.metrics.snapshot(tail)}
