"""Host-side liveness between the ranks of one engine: every rank publishes a heartbeat in the job's key-value
store and checks its peers' before each launch, so that a rank which left (between steps, with nothing in flight)
or stopped beating is noticed on the host and no kernel is enqueued that would wait for it on the device.
The device-side bounded waits remain the second line."""
from __future__ import annotations

import threading
import time
from typing import List, Optional


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.2, limit: float = 2.0, clock=time.time):
        self.store, self.rank, self.world, self.interval, self.limit, self.clock = store, rank, world, interval, limit, clock
        self.stop_flag = threading.Event()
        self.thread: Optional[threading.Thread] = None
        self.beat()

    def beat(self) -> None:
        self.store.set(f"hb/{self.rank}", repr(self.clock()))

    def start(self) -> None:
        def run():
            while not self.stop_flag.wait(self.interval):
                self.beat()
        self.thread = threading.Thread(target=run, name=f"heartbeat-{self.rank}", daemon=True)
        self.thread.start()

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly exit (call between steps, with none of this rank's kernels or collectives in flight)."""
        self.stop_flag.set()
        self.store.set(f"hb/{self.rank}", "left:" + reason)

    def missing(self) -> List[str]:
        """Peers that have left or whose heartbeat is older than the limit, as ``"rank N: why"`` strings."""
        out = []
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"hb/{r}")
                v = v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
            except Exception as ex:
                out.append(f"rank {r}: no heartbeat ({ex})")
                continue
            if v.startswith("left:"):
                out.append(f"rank {r}: {v[5:]}")
            elif now - float(v) > self.limit:
                out.append(f"rank {r}: silent for {now - float(v):.1f} s")
        return out

    def check(self) -> None:
        m = self.missing()
        if m:
            raise RuntimeError("peer failure: " + "; ".join(m))
