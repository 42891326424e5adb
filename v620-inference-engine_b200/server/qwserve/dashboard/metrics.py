"""Rolling time series for the dashboard: fixed-length rings of one sample per second
(reference behaviour: server/qwserve/dashboard/metrics.py:10-106)."""
import collections
import threading
import time
from typing import Dict, List


class Metrics:
    def __init__(self, seconds: int = 600):
        self.seconds = seconds
        self.lock = threading.Lock()
        self.series: Dict[str, collections.deque] = {}
        self.t: collections.deque = collections.deque(maxlen=seconds)
        self.last: Dict[str, float] = {}

    def push(self, sample: Dict[str, float], now: float = None) -> None:
        with self.lock:
            self.t.append(now if now is not None else time.time())
            for k in set(self.series) | set(sample):
                ring = self.series.setdefault(k, collections.deque([0.0] * (len(self.t) - 1), maxlen=self.seconds))
                ring.append(float(sample.get(k, 0.0)))
            self.last = dict(sample)

    def rate(self, key: str, total: float, now: float) -> float:
        """Per-second rate of a monotonically growing counter, from the previous call's value."""
        prev = getattr(self, "_prev", {})
        p = prev.get(key)
        prev[key] = (total, now)
        self._prev = prev
        if p is None or now <= p[1]:
            return 0.0
        return max(0.0, (total - p[0]) / (now - p[1]))

    def snapshot(self, tail: int = 0) -> dict:
        with self.lock:
            n = len(self.t)
            lo = max(0, n - tail) if tail else 0
            return {"t": list(self.t)[lo:], "series": {k: list(v)[lo:] for k, v in self.series.items()}, "last": dict(self.last)}
