"""The fused collectives' word protocol on CPU ranks (threads over shared host memory), for protocol and failure
tests that must not involve a GPU: a rank can be late, skip a push or die, and its peers must time out within their
limit, report who they were waiting for, and stop waiting everywhere once anyone has given up - exactly what the
device code does (``ops/csrc/fuse.cuh``: 8-byte words {payload, sequence}, bounded polls, shared error word,
slots double buffered by the parity of the collective's index).  (The reference has the same abort-on-first-timeout
rule in src/comm/comm.hip:119-139 and tests its protocol only on GPUs.)"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

ERR_WAIT_TIMEOUT = 1


@dataclass
class ErrorWord:
    code: int = 0
    detail: int = 0
    lock: threading.Lock = None

    def report(self, code: int, detail: int) -> None:
        with self.lock:
            if self.code == 0:          # first error wins, like the device's compare-and-swap
                self.code, self.detail = code, detail


class CpuWorld:
    """Receive slots of every rank: ``slots[rank][parity][source rank][word] = (payload, seq)``."""

    def __init__(self, ranks: int, words: int):
        self.ranks, self.words = ranks, words
        self.payload = np.zeros((ranks, 2, ranks, words), dtype=np.float32)
        self.seq = np.zeros((ranks, 2, ranks, words), dtype=np.uint32)
        self.err = [ErrorWord(lock=threading.Lock()) for _ in range(ranks)]


class CpuRank:
    def __init__(self, world: CpuWorld, rank: int, spin_seconds: float = 1.0):
        self.w, self.rank, self.limit = world, rank, spin_seconds
        self.base = 0

    def bump(self, by: int = 4096) -> None:
        self.base += by

    # producer side: this rank's values for collective k go to every rank's slot (all-reduce) ...
    def put_all(self, k: int, values: np.ndarray) -> None:
        seq = np.uint32(self.base + k)
        for d in range(self.w.ranks):
            self.w.payload[d, k & 1, self.rank, :len(values)] = values
            self.w.seq[d, k & 1, self.rank, :len(values)] = seq          # word = payload then sequence: readers check seq

    # ... or column block d of a row goes to rank d (reduce-scatter)
    def put_cols(self, k: int, row: np.ndarray) -> None:
        n = len(row) // self.w.ranks
        seq = np.uint32(self.base + k)
        for d in range(self.w.ranks):
            self.w.payload[d, k & 1, self.rank, :n] = row[d * n:(d + 1) * n]
            self.w.seq[d, k & 1, self.rank, :n] = seq

    # consumer side: the ranks' words added in rank order, or None after a timeout (the error word says for whom)
    def reduce(self, k: int, n: int) -> Optional[np.ndarray]:
        want = np.uint32(self.base + k)
        me = self.w.err[self.rank]
        out = np.zeros(n, dtype=np.float32)
        for r in range(self.w.ranks):
            t0 = time.monotonic()
            while not np.all(self.w.seq[self.rank, k & 1, r, :n] == want):
                if me.code:                                   # someone already gave up: do not wait again
                    return None
                if time.monotonic() - t0 > self.limit:
                    me.report(ERR_WAIT_TIMEOUT, 0x40000000 | (r << 24) | (k & 0xFFFFFF))
                    return None
                time.sleep(0.0002)
            out += self.w.payload[self.rank, k & 1, r, :n]
        return out


def run_ranks(world: CpuWorld, body, spin_seconds: float = 1.0) -> List[object]:
    """Run ``body(rank_object)`` on one thread per rank; returns each rank's result or the exception it raised."""
    res: List[object] = [None] * world.ranks

    def go(i):
        try:
            res[i] = body(CpuRank(world, i, spin_seconds))
        except Exception as ex:         # a rank that dies: its peers find out through their bounded waits
            res[i] = ex
    ts = [threading.Thread(target=go, args=(i,)) for i in range(world.ranks)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return res
