"""ctypes binding of the engine's C API (``libqw_engine.so``) for the server.

One ``Engine`` object = one ``qw_handle``.  All calls except ``failure()`` must come from one thread (the
scheduler's).  ``Tokens`` is a list that caches its int32 array so a long prompt is marshalled once
(reference: server/qwserve/engine.py:10-77)."""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import List, Optional, Sequence, Tuple


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float), ("repetition_penalty", C.c_float),
                ("seed", C.c_uint64)]


class CacheStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("hits", "tokens_restored", "snapshots_saved", "ram_bytes", "disk_bytes", "blocks",
                                          "snapshots", "prompt_tokens", "reused_tokens", "blend_candidate_tokens")]


class SlotTiming(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("restore_s", "prefill_s", "save_s", "pin_wait_s")]


class Media(C.Structure):
    _fields_ = [("hash", C.c_uint64), ("video", C.c_int32), ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32),
                ("patches", C.c_void_p), ("starts", C.c_void_p)]


class StepReq(C.Structure):
    _fields_ = [("slot", C.c_int32), ("pending", C.c_int32), ("budget", C.c_int32), ("flags", C.c_int32), ("sampling", Sampling)]


class Tokens(list):
    """A token list whose ctypes array is built once and reused until the list changes length."""
    _arr = None
    _n = -1

    def array(self):
        if self._arr is None or self._n != len(self):
            self._arr = (C.c_int32 * len(self))(*self)
            self._n = len(self)
        return self._arr


class EngineError(RuntimeError):
    pass


def default_lib() -> str:
    here = os.path.dirname(os.path.abspath(__file__))
    return os.path.normpath(os.path.join(here, "..", "..", "native", "libqw_engine.so"))


class Engine:
    def __init__(self, options: dict, lib_path: Optional[str] = None):
        self.lib = C.CDLL(lib_path or default_lib())
        L = self.lib
        L.qw_open.restype = C.c_void_p
        L.qw_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.qw_error.restype = C.c_char_p
        L.qw_error.argtypes = [C.c_void_p]
        L.qw_slot_capacity.restype = C.c_int64
        for n in ("qw_set_prompt", "qw_begin_prompt"):
            getattr(L, n).restype = C.c_int64
        err = C.create_string_buffer(2048)
        self.h = L.qw_open(json.dumps(options).encode(), err, len(err))
        if not self.h:
            raise EngineError(err.value.decode(errors="replace"))
        self.h = C.c_void_p(self.h)
        self.has_mtp = bool(L.qw_has_mtp(self.h))
        self.has_vision = bool(L.qw_has_vision(self.h))

    def _ck(self, rc):
        if rc < 0:
            raise EngineError((self.lib.qw_error(self.h) or b"").decode(errors="replace"))
        return rc

    def close(self):
        if self.h:
            self.lib.qw_close(self.h)
            self.h = None

    def persist(self):
        self._ck(self.lib.qw_persist(self.h))

    def failure(self) -> str:
        buf = C.create_string_buffer(1024)
        n = self.lib.qw_engine_failure(self.h, buf, len(buf))
        return buf.value.decode(errors="replace") if n else ""

    def set_boundary_token(self, tok: int):
        self._ck(self.lib.qw_set_boundary_token(self.h, tok))

    def cache_stats(self) -> dict:
        s = CacheStats()
        self._ck(self.lib.qw_get_cache_stats(self.h, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in CacheStats._fields_}

    def slot_timing(self, slot: int) -> dict:
        t = SlotTiming()
        self._ck(self.lib.qw_get_slot_timing(self.h, slot, C.byref(t)))
        return {n: float(getattr(t, n)) for n, _ in SlotTiming._fields_}

    def num_slots(self) -> int:
        return self._ck(self.lib.qw_num_slots(self.h))

    def slot_capacity(self, slot: int) -> int:
        return self._ck(self.lib.qw_slot_capacity(self.h, slot))

    def acquire(self, tokens: Tokens, max_new: int, media: Sequence[Media] = ()) -> int:
        if media:
            arr = (Media * len(media))(*media)
            slot = self.lib.qw_acquire_media(self.h, tokens.array(), C.c_int64(len(tokens)), C.c_int64(max_new), arr, len(media))
        else:
            slot = self.lib.qw_acquire(self.h, tokens.array(), C.c_int64(len(tokens)), C.c_int64(max_new))
        if slot < 0:
            msg = (self.lib.qw_error(self.h) or b"").decode(errors="replace")
            if msg:
                raise EngineError(msg)
        return slot

    def release(self, slot: int):
        self._ck(self.lib.qw_release(self.h, slot))

    def prefetch(self, slot: int, tokens: Tokens, media: Sequence[Media] = ()) -> bool:
        arr = (Media * len(media))(*media) if media else None
        return bool(self._ck(self.lib.qw_prefetch(self.h, slot, tokens.array(), C.c_int64(len(tokens)), arr, len(media))))

    def begin_prompt(self, slot: int, tokens: Tokens, media: Sequence[Media] = ()) -> int:
        arr = (Media * len(media))(*media) if media else None
        return self._ck(self.lib.qw_begin_prompt(self.h, slot, tokens.array(), C.c_int64(len(tokens)), arr, len(media)))

    def prefill_some(self, slot: int, max_tokens: int) -> bool:
        return bool(self._ck(self.lib.qw_prefill_some(self.h, slot, C.c_int64(max_tokens))))

    def prefill_batch(self, slots: Sequence[int], max_tokens: Sequence[int]) -> List[bool]:
        """``prefill_some`` for several slots in one call; returns which prompts are in."""
        n = len(slots)
        sl, mt, done = (C.c_int32 * n)(*slots), (C.c_int64 * n)(*max_tokens), (C.c_int32 * n)()
        self._ck(self.lib.qw_prefill_batch(self.h, n, sl, mt, done))
        return [bool(x) for x in done]

    def sample_prompt(self, slot: int, sp: Sampling) -> Tuple[int, float]:
        lp = C.c_float(0)
        return self._ck(self.lib.qw_sample_prompt(self.h, slot, C.byref(sp), C.byref(lp))), lp.value

    def set_stop_tokens(self, slot: int, ids: Sequence[int]):
        arr = (C.c_int32 * len(ids))(*ids)
        self._ck(self.lib.qw_set_stop_tokens(self.h, slot, arr, len(ids)))

    def generate(self, reqs: Sequence[Tuple[int, int, int, int, Sampling]], k: int):
        """reqs: (slot, pending, budget, flags, sampling).  Returns per request (tokens, logprobs, first_row, stopped)."""
        n = len(reqs)
        arr = (StepReq * n)()
        for i, (slot, pending, budget, flags, sp) in enumerate(reqs):
            arr[i] = StepReq(slot, pending, budget, flags, sp)
        toks, lps = (C.c_int32 * (n * (k + 1)))(), (C.c_float * (n * (k + 1)))()
        counts, rows, stopped = (C.c_int32 * n)(), (C.c_int32 * n)(), (C.c_int32 * n)()
        self._ck(self.lib.qw_generate(self.h, n, arr, k, toks, lps, counts, rows, stopped))
        out = []
        for i in range(n):
            c = counts[i]
            out.append((list(toks[i * (k + 1): i * (k + 1) + c]), list(lps[i * (k + 1): i * (k + 1) + c]), rows[i], bool(stopped[i])))
        return out

    def top_logprobs(self, row: int, k: int):
        ids, lps = (C.c_int32 * k)(), (C.c_float * k)()
        n = self._ck(self.lib.qw_top_logprobs(self.h, row, k, ids, lps))
        return list(zip(ids[:n], lps[:n]))

    def top_logprobs_prompt(self, slot: int, k: int):
        ids, lps = (C.c_int32 * k)(), (C.c_float * k)()
        n = self._ck(self.lib.qw_top_logprobs_prompt(self.h, slot, k, ids, lps))
        return list(zip(ids[:n], lps[:n]))
