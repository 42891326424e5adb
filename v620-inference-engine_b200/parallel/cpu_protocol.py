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


# ---------------------------------------------------------------------------------------------------------------------
# The prefill channel's protocol (``ops/csrc/tp.cuh``) on CPU ranks: payloads of any size stored into the peers' receive
# buffers by many producer "CTAs", a ticket per CTA, the last ticket publishes the collective's sequence number to every
# rank's flag, consumers poll (bounded) the flags of all sources and add the parts in rank order.  Sequence numbers count
# the collectives of a kind and travel by value.  A host-side rendezvous (a barrier that every rank's "stream" passes
# before a chunk) is modelled too: it is what keeps a rank whose host was late from costing its peers their bounded wait.
# ---------------------------------------------------------------------------------------------------------------------
class TpWorld:
    def __init__(self, ranks: int, kinds: int, words: int):
        self.ranks, self.kinds, self.words = ranks, kinds, words
        self.parts = np.zeros((ranks, kinds, ranks, words), dtype=np.float32)          # [receiver][kind][source][word]
        self.flags = np.zeros((ranks, kinds, ranks), dtype=np.uint32)                  # [receiver][kind][source]
        self.err = [ErrorWord(lock=threading.Lock()) for _ in range(ranks)]
        self.barrier = threading.Barrier(ranks)


class TpRank:
    def __init__(self, world: TpWorld, rank: int, spin_seconds: float = 1.0):
        self.w, self.rank, self.limit = world, rank, spin_seconds
        self.seq = [0] * world.kinds                  # host-side counters, handed to the "kernels" by value
        self.ticket = [0] * world.kinds

    def rendezvous(self, timeout: float = 30.0) -> bool:
        """What a one-element all-reduce on the stream does for the chunk that follows: nobody starts before all are here."""
        try:
            self.w.barrier.wait(timeout)
            return True
        except threading.BrokenBarrierError:
            return False

    def send(self, kind: int, values: np.ndarray, ctas: int = 4) -> int:
        """All-reduce / all-gather producer: ``ctas`` producers store slices of ``values`` into every rank's part of this
        rank, each takes a ticket, the last one publishes.  Returns the collective's sequence number."""
        self.seq[kind] += 1
        seq = self.seq[kind]
        n = len(values)
        step = (n + ctas - 1) // ctas
        for c in range(ctas):
            lo, hi = c * step, min(n, (c + 1) * step)
            for d in range(self.w.ranks):
                self.w.parts[d, kind, self.rank, lo:hi] = values[lo:hi]
            self.ticket[kind] += 1                    # after the CTA's stores (the device fences system-wide here)
            if self.ticket[kind] == ctas:
                self.ticket[kind] = 0
                for d in range(self.w.ranks):
                    self.w.flags[d, kind, self.rank] = np.uint32(seq)          # release store of the sequence number
        return seq

    def receive(self, kind: int, n: int, seq: int) -> Optional[np.ndarray]:
        """Consumer: bounded wait for every source's flag to reach ``seq``, then the parts added in rank order."""
        err = self.w.err[self.rank]
        t0 = time.monotonic()
        for r in range(self.w.ranks):
            while ((int(self.w.flags[self.rank, kind, r]) - seq + (1 << 31)) % (1 << 32)) - (1 << 31) < 0:          # (int32)(flag - seq) < 0
                if err.code:                          # someone already gave up: do not sit out the limit again
                    return None
                if time.monotonic() - t0 > self.limit:
                    err.report(ERR_WAIT_TIMEOUT, 0x20000000 | (r << 24) | (seq & 0xffffff))
                    return None
                time.sleep(0)
        out = np.zeros(n, dtype=np.float32)
        for r in range(self.w.ranks):
            out += self.w.parts[self.rank, kind, r, :n]
        return out


def run_tp_ranks(world: TpWorld, body, spin_seconds: float = 1.0) -> List[object]:
    res: List[object] = [None] * world.ranks

    def go(i):
        res[i] = body(TpRank(world, i, spin_seconds))
    ts = [threading.Thread(target=go, args=(i,)) for i in range(world.ranks)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return res
