"""Environment-gated host timers (``QW_TRACE``) and prefill profiling (``QW_PROFILE``).

* ``StepTrace``: per row count, the host preparation / launch / copy-back / total milliseconds of decode steps,
  printed every 50 steps (reference: src/engine/decode.hip:183-199,453-456).
* ``PhaseTrace``: named phases of one ``generate`` call and its sampling fallbacks (src/session/generate.cpp:93-116).
* ``ChunkProfile``: CUDA-event time of every prefill chunk (src/engine/prefill.hip:47,491-495).
All of them cost nothing when their switch is off: the objects are created disabled and every method returns at once."""
from __future__ import annotations

import collections
import sys
import time
from typing import Callable, Dict, List, Optional


def _log(msg: str) -> None:
    print(msg, file=sys.stderr, flush=True)


class StepTrace:
    def __init__(self, enabled: bool, every: int = 50, log: Callable[[str], None] = _log):
        self.on, self.every, self.log = enabled, every, log
        self.acc: Dict[int, List[float]] = collections.defaultdict(lambda: [0, 0.0, 0.0, 0.0, 0.0])
        self.t0 = self.t1 = self.t2 = 0.0

    def begin(self):
        if self.on:
            self.t0 = time.perf_counter()

    def launched(self):          # host preparation done, the step is enqueued
        if self.on:
            self.t1 = time.perf_counter()

    def enqueued(self):          # launch call returned
        if self.on:
            self.t2 = time.perf_counter()

    def end(self, rows: int):    # results are on the host
        if not self.on:
            return
        t3 = time.perf_counter()
        a = self.acc[rows]
        a[0] += 1
        a[1] += self.t1 - self.t0
        a[2] += self.t2 - self.t1
        a[3] += t3 - self.t2
        a[4] += t3 - self.t0
        if a[0] >= self.every:
            n = a[0]
            self.log(f"[trace] decode rows={rows}: prep {1e3 * a[1] / n:.3f} ms, launch {1e3 * a[2] / n:.3f} ms, "
                     f"wait+copy {1e3 * a[3] / n:.3f} ms, total {1e3 * a[4] / n:.3f} ms over {n} steps")
            self.acc[rows] = [0, 0.0, 0.0, 0.0, 0.0]


class PhaseTrace:
    def __init__(self, enabled: bool, name: str = "generate", every: int = 50, log: Callable[[str], None] = _log):
        self.on, self.name, self.every, self.log = enabled, name, every, log
        self.ms: Dict[str, float] = collections.defaultdict(float)
        self.counts: Dict[str, int] = collections.defaultdict(int)
        self.calls = 0
        self.t = 0.0

    def start(self):
        if self.on:
            self.t = time.perf_counter()

    def mark(self, phase: str):
        if self.on:
            now = time.perf_counter()
            self.ms[phase] += 1e3 * (now - self.t)
            self.t = now

    def count(self, what: str, n: int = 1):
        if self.on:
            self.counts[what] += n

    def finish(self):
        if not self.on:
            return
        self.calls += 1
        if self.calls >= self.every:
            parts = ", ".join(f"{k} {v / self.calls:.3f}" for k, v in self.ms.items())
            extra = ", ".join(f"{k}={v}" for k, v in self.counts.items())
            self.log(f"[trace] {self.name}: ms per call: {parts}" + (f"; {extra}" if extra else "") + f" over {self.calls} calls")
            self.ms.clear()
            self.counts.clear()
            self.calls = 0


class ChunkProfile:
    """CUDA-event time of prefill chunks; ``summary()`` after the prompt."""

    def __init__(self, enabled: bool, log: Callable[[str], None] = _log):
        self.on, self.log = enabled, log
        self.events = []

    def begin(self):
        if not self.on:
            return None
        import torch
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def end(self, start, tokens: int):
        if not self.on or start is None:
            return
        import torch
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((start, e, tokens))

    def summary(self, label: str = "prefill") -> Optional[str]:
        if not self.on or not self.events:
            return None
        import torch
        torch.cuda.synchronize()
        ms = [(a.elapsed_time(b), n) for a, b, n in self.events]
        self.events.clear()
        tot, toks = sum(m for m, _ in ms), sum(n for _, n in ms)
        line = (f"[profile] {label}: {len(ms)} chunks, {toks} tokens, {tot:.1f} ms on the device "
                f"({toks / max(tot, 1e-6) * 1e3:.0f} tok/s); per chunk ms: " + " ".join(f"{m:.1f}" for m, _ in ms[:16]))
        self.log(line)
        return line
