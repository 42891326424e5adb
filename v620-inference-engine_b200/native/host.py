"""ctypes bindings of the native host runtime (``libqw_host.so``)."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import build as nbuild

_lib = None
P, LL, ULL, I = C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_int


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float), ("repetition_penalty", C.c_float),
                ("seed", C.c_uint64)]

    @staticmethod
    def make(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, presence_penalty=0.0, frequency_penalty=0.0,
             repetition_penalty=1.0, seed=0) -> "Sampling":
        return Sampling(temperature, top_p, top_k, min_p, presence_penalty, frequency_penalty, repetition_penalty, seed)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        nbuild.build()
        L = C.CDLL(nbuild.HOST_LIB)
        sig = {
            "qwh_last_error": (C.c_char_p, []),
            "qwh_ngram_new": (P, [I, I, I, I, LL, ULL, I, I]), "qwh_ngram_free": (None, [P]), "qwh_ngram_total_rows": (LL, [P]),
            "qwh_ngram_sizes": (I, [P, P, P, P]), "qwh_ngram_ids": (I, [P, P, I, P, I, P]),
            "qwh_spec_new": (P, [I, C.c_double, C.c_double, C.c_double, I, I, I]), "qwh_spec_free": (None, [P]), "qwh_spec_slots": (P, [P]),
            "qwh_spec_draft_count": (I, [P, I, I]), "qwh_spec_best_rate": (C.c_double, [P, C.c_double, I, P]),
            "qwh_spec_plan": (I, [P, I, P, P, P, P, I, I, I, I, I, P, P]), "qwh_spec_note_plain_step": (I, [P, I]),
            "qwh_spec_accept": (I, [P, I, P, P, I, P, I, I]),
            "qwh_choose_slot": (I, [I, P, P, P, P, LL]), "qwh_start_way": (I, [LL, LL, LL]),
            "qwh_capture_point": (LL, [P, LL, LL, LL, LL, I, LL]), "qwh_best_snapshot": (I, [I, P, P, LL, LL]),
            "qwh_sampler_full_sort": (None, [I]), "qwh_pool_new": (P, [I]), "qwh_pool_free": (None, [P]), "qwh_pool_size": (I, [P]), "qwh_pool_check": (LL, [P, LL, LL, I]),
            "qwh_ple_open": (P, [C.c_char_p, I]), "qwh_ple_free": (None, [P]), "qwh_ple_rows": (LL, [P]), "qwh_ple_layout": (I, [P]),
            "qwh_ple_gather": (I, [P, P, I, I, P, P]), "qwh_ple_pin": (I, [P, I, I]),
            "qwh_st_open": (P, [C.c_char_p]), "qwh_st_add": (I, [P, C.c_char_p]), "qwh_st_free": (None, [P]), "qwh_st_count": (I, [P]),
            "qwh_st_info": (I, [P, C.c_char_p, P, P, P, P, P]),
            "qwh_store_new": (P, [ULL, C.c_uint, ULL, C.c_char_p, ULL]), "qwh_store_free": (None, [P]), "qwh_store_root": (ULL, []),
            "qwh_block_key": (ULL, [ULL, P, I]), "qwh_store_save_block": (ULL, [P, ULL, LL, P, I, P, ULL]),
            "qwh_store_save_snapshot": (I, [P, ULL, P, ULL, P, I, I]), "qwh_store_lookup": (I, [P, P, LL, P, I, P]),
            "qwh_store_get": (LL, [P, ULL, I, P, ULL, P, I, P]), "qwh_store_block_info": (I, [P, ULL, P, P, P, P, P]),
            "qwh_store_note_restore": (None, [P, ULL, LL]), "qwh_store_flush": (None, [P]), "qwh_store_thin": (I, [P, LL]),
            "qwh_store_stats": (None, [P, P]), "qwh_store_prefetch": (I, [P, P, I, I]), "qwh_store_loads_pending": (I, [P]),
            "qwh_rng_new": (P, [ULL]), "qwh_rng_free": (None, [P]), "qwh_sample": (I, [P, I, P, P, LL, LL, P, P]),
            "qwh_top_logprobs": (I, [P, I, I, P, P]), "qwh_lse": (C.c_float, [P, I]),
            "qwh_chunk": (I, [P, LL, I, P, P, P, I]),
            "qwh_pinned_new": (P, [ULL, ULL, I, I, I, I]), "qwh_pinned_free": (None, [P]), "qwh_pinned_reserve": (None, [P, I]),
            "qwh_pinned_get": (P, [P]), "qwh_pinned_put": (I, [P, P]), "qwh_pinned_unit_bytes": (ULL, [P]),
            "qwh_pinned_stats": (None, [P, P, P, P]), "qwh_numa_nodes": (I, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _err() -> str:
    return (lib().qwh_last_error() or b"").decode()


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


class NgramHasher:
    def __init__(self, cfg):
        self.cfg = cfg
        self.h = lib().qwh_ngram_new(cfg.vocab, cfg.eos, cfg.ngram, cfg.ngram_heads, cfg.ngram_vocab_base, cfg.ple_seed,
                                     cfg.image_pad, cfg.video_pad)
        if not self.h:
            raise RuntimeError(_err())
        self.total_rows = lib().qwh_ngram_total_rows(self.h)

    def ids_for(self, history: Sequence[int], tokens: Sequence[int]) -> np.ndarray:
        h, t = _i32(history), _i32(tokens)
        out = np.zeros((len(t), self.cfg.ngram_heads), dtype=np.int64)
        if lib().qwh_ngram_ids(self.h, h.ctypes.data, len(h), t.ctypes.data, len(t), out.ctypes.data) != 0:
            raise RuntimeError(_err())
        return out

    def __del__(self):
        if getattr(self, "h", None):
            lib().qwh_ngram_free(self.h)
            self.h = None


class PleTableNative:
    def __init__(self, path: str, width: int, threads: int = 8):
        self.t = lib().qwh_ple_open(path.encode(), width)
        if not self.t:
            raise RuntimeError(_err())
        self.width = width
        self.pool = lib().qwh_pool_new(threads)
        self.rows = lib().qwh_ple_rows(self.t)

    def gather(self, ids: np.ndarray) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        T, heads = ids.shape
        out = np.empty((T, heads * self.width), dtype=np.float32)
        if lib().qwh_ple_gather(self.t, ids.ctypes.data, T, heads, out.ctypes.data, self.pool) != 0:
            raise RuntimeError(_err())
        return out

    def pin(self, lock: bool = True, wait: bool = False):
        lib().qwh_ple_pin(self.t, int(lock), int(wait))

    def __del__(self):
        if getattr(self, "t", None):
            lib().qwh_ple_free(self.t)
            lib().qwh_pool_free(self.pool)
            self.t = None


class BlockStore:
    """Prefix cache over opaque payloads; see src/block_store.hpp."""
    BLOCK = 256

    def __init__(self, layout: int, ranks: int, ram_budget: int, disk_dir: Optional[str] = None, disk_budget: int = 0):
        self.s = lib().qwh_store_new(layout, ranks, ram_budget, disk_dir.encode() if disk_dir else None, disk_budget)
        if not self.s:
            raise RuntimeError(_err())
        self.root = lib().qwh_store_root()

    def close(self):
        if getattr(self, "s", None) and lib is not None:      # `lib` is gone when the interpreter is shutting down
            lib().qwh_store_free(self.s)
            self.s = None

    __del__ = close

    @staticmethod
    def key(parent: int, tokens: Sequence[int]) -> int:
        t = _i32(tokens)
        return lib().qwh_block_key(parent, t.ctypes.data, len(t))

    def save_block(self, parent: int, start: int, tokens: Sequence[int], kv: bytes) -> int:
        t = _i32(tokens)
        buf = (C.c_char * len(kv)).from_buffer_copy(kv)
        return lib().qwh_store_save_block(self.s, parent, start, t.ctypes.data, len(t), C.addressof(buf), len(kv))

    def save_block_from(self, parent: int, start: int, tokens: Sequence[int], addr: int, nbytes: int) -> int:
        """``save_block`` with the payload given by address (a pinned unit the engine exported into): no intermediate copy."""
        t = _i32(tokens)
        return lib().qwh_store_save_block(self.s, parent, start, t.ctypes.data, len(t), addr, nbytes)

    def get_into(self, key: int, out: np.ndarray) -> int:
        """Copy a block's KV payload into ``out`` (uint8, e.g. a pinned unit).  Returns its size, or -1 when it is gone."""
        nl = C.c_int(0)
        size = lib().qwh_store_get(self.s, key, 0, None, 0, None, 0, C.byref(nl))
        if size < 0 or size > out.nbytes:
            return -1
        lib().qwh_store_get(self.s, key, 0, out.ctypes.data, size, None, 0, C.byref(nl))
        return int(size)

    def prefetch(self, keys: Sequence[int], last_snapshot: bool = True) -> int:
        """Queue background reads of the blocks' payloads that are only on disk (and of the last block's snapshot).  Returns
        the number of reads queued; ``loads_pending()`` tells when they are done."""
        if not keys:
            return 0
        arr = (C.c_ulonglong * len(keys))(*[int(k) for k in keys])
        return int(lib().qwh_store_prefetch(self.s, arr, len(keys), int(last_snapshot)))

    def loads_pending(self) -> int:
        return int(lib().qwh_store_loads_pending(self.s))

    def save_snapshot(self, key: int, snap: bytes, logits: Optional[np.ndarray] = None, anchor: bool = False) -> bool:
        buf = (C.c_char * len(snap)).from_buffer_copy(snap)
        lg = None if logits is None else np.ascontiguousarray(logits, dtype=np.float32)
        return lib().qwh_store_save_snapshot(self.s, key, C.addressof(buf), len(snap), None if lg is None else lg.ctypes.data,
                                             0 if lg is None else lg.size, int(anchor)) == 0

    def save_snapshot_from(self, key: int, addr: int, nbytes: int, anchor: bool = False) -> bool:
        """``save_snapshot`` with the payload given by address (pinned memory the engine exported into)."""
        return lib().qwh_store_save_snapshot(self.s, key, addr, nbytes, None, 0, int(anchor)) == 0

    def get_snapshot_into(self, key: int, out: np.ndarray) -> int:
        """Copy a block's snapshot payload into ``out`` (uint8).  Returns its size, or -1 when there is none or it does not fit."""
        nl = C.c_int(0)
        size = lib().qwh_store_get(self.s, key, 1, None, 0, None, 0, C.byref(nl))
        if size < 0 or size > out.nbytes:
            return -1
        lib().qwh_store_get(self.s, key, 1, out.ctypes.data, size, None, 0, C.byref(nl))
        return int(size)

    def lookup(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        t = _i32(tokens)
        keys = (C.c_ulonglong * (len(t) // self.BLOCK + 2))()
        depth = C.c_int(0)
        n = lib().qwh_store_lookup(self.s, t.ctypes.data, len(t), keys, len(keys), C.byref(depth))
        return [int(keys[i]) for i in range(max(n, 0))], depth.value

    def get(self, key: int, snapshot: bool = False):
        nl = C.c_int(0)
        size = lib().qwh_store_get(self.s, key, int(snapshot), None, 0, None, 0, C.byref(nl))
        if size < 0:
            return None
        buf = C.create_string_buffer(size)
        lg = np.empty(nl.value, dtype=np.float32)
        lib().qwh_store_get(self.s, key, int(snapshot), buf, size, lg.ctypes.data if nl.value else None, nl.value, C.byref(nl))
        return (buf.raw, lg) if snapshot else buf.raw

    def info(self, key: int):
        st, nt, hs, ram, dk = LL(0), I(0), I(0), I(0), I(0)
        if lib().qwh_store_block_info(self.s, key, C.byref(st), C.byref(nt), C.byref(hs), C.byref(ram), C.byref(dk)) != 0:
            return None
        return {"start": st.value, "ntok": nt.value, "has_snap": bool(hs.value), "in_ram": bool(ram.value), "on_disk": bool(dk.value)}

    def note_restore(self, key: int, tokens: int):
        lib().qwh_store_note_restore(self.s, key, tokens)

    def flush(self):
        lib().qwh_store_flush(self.s)

    def thin(self, gap: int) -> int:
        return lib().qwh_store_thin(self.s, gap)

    def stats(self) -> dict:
        out = (C.c_ulonglong * 7)()
        lib().qwh_store_stats(self.s, out)
        names = ["hits", "tokens_restored", "snapshots_saved", "ram_bytes", "disk_bytes", "blocks", "snapshots"]
        return dict(zip(names, [int(x) for x in out]))


START_RESET, START_IN_PLACE, START_DEVICE_SNAPSHOT, START_STORE = 0, 1, 2, 3


def choose_slot(busy: Sequence[bool], capacity: Sequence[int], kept: Sequence[int], used: Sequence[int], need: int) -> int:
    """The free slot that holds ``need`` tokens and keeps the most of the prompt, then the least recently used (-1: none)."""
    b = np.asarray(busy, dtype=np.uint8)
    c, k, u = (np.asarray(x, dtype=np.int64) for x in (capacity, kept, used))
    return int(lib().qwh_choose_slot(len(b), b.ctypes.data, c.ctypes.data, k.ctypes.data, u.ctypes.data, int(need)))


def start_way(keep: int, snapshot: int, stored: int) -> int:
    """How a prompt starts: one of START_RESET / START_IN_PLACE / START_DEVICE_SNAPSHOT / START_STORE (src/slot_logic.hpp)."""
    return int(lib().qwh_start_way(int(keep), int(snapshot), int(stored)))


def capture_point(piece: Sequence[int], first: int, prompt_len: int, done: int, end: int, last_capture: int, boundary: int, min_gap: int) -> int:
    """Where the prefill piece [done, end) should end for a device snapshot at a message boundary.  ``piece`` holds the
    prompt's tokens from position ``first`` on (only the part the search can look at needs to be passed)."""
    t = _i32(piece)
    r = lib().qwh_capture_point(t.ctypes.data, min(int(prompt_len), int(first) + len(t)) - int(first), int(done) - int(first), int(end) - int(first),
                                int(last_capture) - int(first), int(boundary), int(min_gap))
    return int(r) + int(first)


def best_snapshot(depths: Sequence[int], has_logits: Sequence[bool], common: int, prompt_len: int) -> int:
    d, h = np.asarray(depths, dtype=np.int64), np.asarray(has_logits, dtype=np.uint8)
    return int(lib().qwh_best_snapshot(len(d), d.ctypes.data, h.ctypes.data, int(common), int(prompt_len)))


class SpecSlot(C.Structure):
    """One slot's speculative-decoding state as the native planner keeps it (src/spec_planner.hpp); the session reads
    and writes these fields in place."""
    _fields_ = [("accept", C.c_double), ("plain_left", C.c_int32), ("plain_stretch", C.c_int32)]


class SpecPlanner:
    """How many drafts each request of a step gets, the stretches without drafts, and what is kept of a verified run:
    src/spec_planner.hpp."""
    ERRORS = {-1: "a request needs a budget of at least one token", -2: "slot {slot} is full", -3: "more requests than rows in a step"}

    def __init__(self, slots: int, base: float, beta: float, probe_accept: float, plain_first: int, plain_grow: int, plain_max: int):
        self.h = lib().qwh_spec_new(slots, base, beta, probe_accept, plain_first, plain_grow, plain_max)
        self.n = slots
        self.slots = (SpecSlot * slots).from_address(lib().qwh_spec_slots(self.h))       # the planner's own memory

    def best_rate(self, a: float, k_max: int) -> Tuple[float, int]:
        k = C.c_int(0)
        r = lib().qwh_spec_best_rate(self.h, a, k_max, C.byref(k))
        return float(r), k.value

    def draft_count(self, slot: int, k_max: int) -> int:
        return int(lib().qwh_spec_draft_count(self.h, slot, k_max))

    def plan(self, slots: Sequence[int], budgets: Sequence[int], room: Sequence[int], can_draft: Sequence[bool], k: int, max_drafts: int,
             max_run: int, max_rows: int, forced: bool) -> List[int]:
        n = len(slots)
        sl, bu, ro = _i32(slots), np.asarray(budgets, dtype=np.int64), np.asarray(room, dtype=np.int64)
        cd = np.asarray(can_draft, dtype=np.uint8)
        want, bad = np.zeros(max(n, 1), dtype=np.int32), C.c_int(-1)
        rc = lib().qwh_spec_plan(self.h, n, sl.ctypes.data, bu.ctypes.data, ro.ctypes.data, cd.ctypes.data, int(k), int(max_drafts), int(max_run),
                                 int(max_rows), int(bool(forced)), want.ctypes.data, C.byref(bad))
        if rc != 0:
            raise ValueError(self.ERRORS[rc].format(slot=slots[bad.value] if 0 <= bad.value < n else "?"))
        return [int(x) for x in want[:n]]

    def note_plain_step(self, slot: int) -> int:
        return int(lib().qwh_spec_note_plain_step(self.h, slot))

    def accept(self, slot: int, sampled: Sequence[int], drafts: Sequence[int], stop: Sequence[int], forced: Optional[int]) -> int:
        s, d, st = _i32(sampled), _i32(drafts), _i32(stop)
        return int(lib().qwh_spec_accept(self.h, slot, s.ctypes.data, d.ctypes.data, len(d), st.ctypes.data, len(st), -1 if forced is None else int(forced)))

    def __del__(self):
        if getattr(self, "h", None) and lib is not None:
            self.slots = None
            lib().qwh_spec_free(self.h)
            self.h = None


class HostSampler:
    def __init__(self, seed: int = 0):
        self.rng = lib().qwh_rng_new(seed)

    def sample(self, logits: np.ndarray, p: Sampling, hist: Sequence[int] = (), prompt_end: int = 0) -> Tuple[int, float]:
        lg = np.ascontiguousarray(logits, dtype=np.float32)
        h = _i32(hist)
        lp = C.c_float(0)
        tok = lib().qwh_sample(lg.ctypes.data, lg.size, C.byref(p), h.ctypes.data, len(h), prompt_end, self.rng, C.byref(lp))
        if tok < 0:
            raise RuntimeError(_err())
        return tok, lp.value

    @staticmethod
    def top_logprobs(logits: np.ndarray, k: int):
        lg = np.ascontiguousarray(logits, dtype=np.float32)
        ids, lps = np.zeros(k, dtype=np.int32), np.zeros(k, dtype=np.float32)
        n = lib().qwh_top_logprobs(lg.ctypes.data, lg.size, k, ids.ctypes.data, lps.ctypes.data)
        return ids[:n], lps[:n]

    def __del__(self):
        if getattr(self, "rng", None) and lib is not None:
            lib().qwh_rng_free(self.rng)
            self.rng = None


def chunk_prompt(tokens: Sequence[int], boundary: int):
    t = _i32(tokens)
    cap = len(t) // 128 + 8
    st, ln, hs = np.zeros(cap, dtype=np.int64), np.zeros(cap, dtype=np.int64), np.zeros(cap, dtype=np.uint64)
    n = lib().qwh_chunk(t.ctypes.data, len(t), boundary, st.ctypes.data, ln.ctypes.data, hs.ctypes.data, cap)
    return [(int(st[i]), int(ln[i]), int(hs[i])) for i in range(min(n, cap))]


class PinnedPool:
    """Pinned host memory in fixed units from background-pinned arenas (``native/src/pinned_pool.hpp``).  ``get()`` returns
    a uint8 numpy view of one unit; give it back with ``put``.  With ``use_cuda`` the arenas are also registered with the
    CUDA runtime when it is loaded in the process, so copies from / to the units are asynchronous."""
    POLICIES = {"process": 0, "bind": 1, "preferred": 2, "interleave": 3, "auto": 0}

    def __init__(self, unit_bytes: int, arena_bytes: int = 256 << 20, standing_units: int = 2, use_cuda: bool = False,
                 policy: str = "process", node: int = -1):
        self.p = lib().qwh_pinned_new(unit_bytes, arena_bytes, standing_units, int(use_cuda), self.POLICIES[policy], node)
        if not self.p:
            raise RuntimeError(_err())
        self.unit_bytes = int(lib().qwh_pinned_unit_bytes(self.p))
        self._out = {}

    def reserve(self, n: int) -> None:
        lib().qwh_pinned_reserve(self.p, n)

    def get(self) -> np.ndarray:
        addr = lib().qwh_pinned_get(self.p)
        if not addr:
            raise RuntimeError(_err())
        a = np.ctypeslib.as_array(C.cast(addr, C.POINTER(C.c_uint8)), shape=(self.unit_bytes,))
        self._out[a.ctypes.data] = addr
        return a

    def put(self, a: np.ndarray) -> None:
        addr = self._out.pop(a.ctypes.data)
        if lib().qwh_pinned_put(self.p, addr) != 0:
            raise RuntimeError(_err())

    def stats(self) -> dict:
        i5, d2, x2 = (C.c_longlong * 5)(), (C.c_double * 2)(), (C.c_int * 2)()
        lib().qwh_pinned_stats(self.p, i5, d2, x2)
        return {"arenas": i5[0], "units_total": i5[1], "units_free": i5[2], "gets": i5[3], "waits": i5[4], "wait_seconds": d2[0],
                "pin_seconds": d2[1], "cuda_registered": bool(x2[0]), "numa_node": x2[1]}

    def close(self) -> None:
        if getattr(self, "p", None) and lib is not None:
            lib().qwh_pinned_free(self.p)
            self.p = None

    __del__ = close


def numa_nodes() -> int:
    return int(lib().qwh_numa_nodes())
