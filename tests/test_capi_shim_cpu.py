"""The C ABI end to end without a GPU: the server's ctypes binding -> libqw_engine.so (the C shim) -> capi_impl.CApi ->
a scripted session.  Every one of the 29 functions is called through C; the scripted session records what arrived and
returns known values, so argument order, pointer marshalling, struct layouts, return conventions (>= 0 ok, -1 + qw_error)
and the error path are checked where they are implemented - in the shim and the two Python sides of it."""
import ctypes as C
import os
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SERVER = os.path.join(ROOT, "v620-inference-engine_b200", "server")
if SERVER not in sys.path:
    sys.path.insert(0, SERVER)


class ScriptedSession:
    """What CApi / SessionOps call on a Session, recording the arguments."""

    def __init__(self):
        self.calls = []
        self.store = types.SimpleNamespace(flush=lambda: self.calls.append(("flush",)))
        self.e = types.SimpleNamespace(mtp=True, dm=types.SimpleNamespace(check_error=self._check))
        self.device_error = ""
        self.pending_loads = 2

    def _check(self):
        if self.device_error:
            raise RuntimeError(self.device_error)

    def _rec(self, *a):
        self.calls.append(a)

    def persist(self): self._rec("persist")
    def set_boundary_token(self, t): self._rec("boundary", t)
    def num_slots(self): return 3
    def slot_capacity(self, s): return 131072 + s

    def acquire(self, toks, max_new):
        self._rec("acquire", list(toks), max_new)
        if 666 in toks:
            raise ValueError("this prompt is refused")
        return -1 if len(toks) > 100 else 1

    def release(self, s): self._rec("release", s)

    def begin_prompt(self, s, toks):
        self._rec("begin", s, list(toks))
        return 5000000000 if s == 2 else 256                 # more than 32 bits must survive the trip

    def prefetch(self, toks): self._rec("prefetch", list(toks))
    def loads_pending(self): return self.pending_loads

    def prefill_some(self, s, n):
        self._rec("prefill_some", s, n)
        return n >= 1000

    def sample_prompt(self, s, sp):
        self._rec("sample_prompt", s, round(sp.temperature, 3), sp.top_k, round(sp.top_p, 3), sp.seed, round(sp.repetition_penalty, 3))
        return 4242, -0.75

    def decode(self, slots, tokens): self._rec("decode", list(slots), list(tokens))

    def sample_row(self, row, sp):
        self._rec("sample_row", row, sp.top_k)
        return 77 + row, -1.5

    def set_stop_tokens(self, s, ids): self._rec("stop", s, list(ids))

    def generate(self, reqs, k):
        self._rec("generate", [(r.slot, r.pending, r.budget, r.flags, r.sampling.top_k) for r in reqs], k)
        out, row = [], 0
        for i, r in enumerate(reqs):
            toks = [r.pending + j + 1 for j in range(min(k + 1, i + 1))]
            out.append(types.SimpleNamespace(tokens=toks, logprobs=[-0.1 * (j + 1) for j in range(len(toks))], first_row=row, stopped=(i == 1)))
            row += len(toks)
        return out

    def top_logprobs(self, row, k): return [10 + row, 11, 12][:k], [-0.5, -1.5, -2.5][:k]
    def top_logprobs_prompt(self, slot, k): return [20 + slot, 21][:k], [-0.25, -1.25][:k]

    def cache_stats(self):
        return dict(hits=3, tokens_restored=768, snapshots_saved=5, ram_bytes=1 << 33, disk_bytes=1 << 35, blocks=9, snapshots=4,
                    prompt_tokens=1000, reused_tokens=600, blend_candidate_tokens=128)

    def slot_timing(self, slot):
        return dict(restore_s=0.25, prefill_s=1.5 + slot, save_s=0.125, pin_wait_s=0.0)


@pytest.fixture
def opened(monkeypatch):
    from qwb200 import capi_impl
    from qwb200.native import build as nbuild
    nbuild.build()
    ses = ScriptedSession()
    seen = {}

    def fake_build_ops(o, rank, world, port):
        seen["options"] = o
        return capi_impl.SessionOps(ses, None)
    monkeypatch.setattr(capi_impl, "build_ops", fake_build_ops)
    from qwserve import engine as E
    eng = E.Engine({"synthetic": "tiny", "slots": [4096, 4096], "prefill_chunk": 512}, nbuild.ENGINE_LIB)
    yield eng, ses, seen, E
    eng.close()


def test_every_function_of_the_c_abi(opened):
    eng, ses, seen, E = opened
    assert seen["options"] == {"synthetic": "tiny", "slots": [4096, 4096], "prefill_chunk": 512}      # the JSON arrived whole
    assert eng.has_mtp is True and eng.has_vision is False
    assert eng.num_slots() == 3 and eng.slot_capacity(2) == 131074
    eng.set_boundary_token(248046)
    eng.persist()
    assert ("boundary", 248046) in ses.calls and ("persist",) in ses.calls
    # prompts: tokens cross as an int32 array, 64-bit lengths and results
    toks = E.Tokens([5, 6, 7, 2**31 - 1, 0])
    assert eng.acquire(toks, 99) == 1 and ses.calls[-1] == ("acquire", [5, 6, 7, 2**31 - 1, 0], 99)
    assert eng.acquire(E.Tokens(range(200)), 1) == -1                     # no slot: -1 without an error
    with pytest.raises(E.EngineError, match="this prompt is refused"):    # a refusal: -1 with the message in qw_error
        eng.acquire(E.Tokens([1, 666]), 1)
    assert eng.begin_prompt(1, toks) == 256 and ses.calls[-1] == ("begin", 1, [5, 6, 7, 2**31 - 1, 0])
    assert eng.begin_prompt(2, toks) == 5000000000
    assert eng.prefetch(1, toks) is True and ses.calls[-1][0] == "prefetch"
    ses.pending_loads = 0
    assert eng.prefetch(1, toks) is False
    assert eng.prefill_some(1, 512) is False and eng.prefill_some(1, 1 << 40) is True and ses.calls[-1] == ("prefill_some", 1, 1 << 40)
    assert eng.prefill_batch([0, 2, 1], [2048, 16, 1000]) == [True, False, True]
    eng.set_stop_tokens(1, [248044, 248046])
    assert ses.calls[-1] == ("stop", 1, [248044, 248046])
    # sampling parameters cross as a struct
    sp = E.Sampling(temperature=0.7, top_p=0.8, top_k=20, min_p=0.0, presence_penalty=1.5, frequency_penalty=0.0, repetition_penalty=1.05, seed=2**40 + 3)
    assert eng.sample_prompt(1, sp) == (4242, -0.75)
    assert ses.calls[-1] == ("sample_prompt", 1, 0.7, 20, 0.8, 2**40 + 3, 1.05)
    # plain decode + per-row sampling
    L, h = eng.lib, eng.h
    sl, tk = (C.c_int32 * 2)(0, 1), (C.c_int32 * 2)(11, 22)
    assert L.qw_decode(h, 2, sl, tk) == 0 and ses.calls[-1] == ("decode", [0, 1], [11, 22])
    lp = C.c_float(0)
    assert L.qw_sample_row(h, 1, C.byref(sp), C.byref(lp)) == 78 and lp.value == -1.5
    # a generation step for three requests: ragged results in (k + 1)-wide rows
    outs = eng.generate([(0, 100, 8, 0, sp), (1, 200, 8, E.QW_STEP_LOGITS if hasattr(E, "QW_STEP_LOGITS") else 1, sp), (2, 300, 8, 0, sp)], 2)
    assert ses.calls[-1][0] == "generate" and ses.calls[-1][2] == 2 and [r[:3] for r in ses.calls[-1][1]] == [(0, 100, 8), (1, 200, 8), (2, 300, 8)]
    assert [o[0] for o in outs] == [[101], [201, 202], [301, 302, 303]]
    assert [o[2] for o in outs] == [0, 1, 3] and [o[3] for o in outs] == [False, True, False]
    assert abs(outs[2][1][2] + 0.3) < 1e-6
    assert eng.top_logprobs(2, 3) == [(12, -0.5), (11, -1.5), (12, -2.5)]
    assert eng.top_logprobs_prompt(1, 5) == [(21, -0.25), (21, -1.25)]
    # structs written by the engine
    st = eng.cache_stats()
    assert st["ram_bytes"] == 1 << 33 and st["disk_bytes"] == 1 << 35 and st["reused_tokens"] == 600 and st["blend_candidate_tokens"] == 128
    tm = eng.slot_timing(2)
    assert tm["prefill_s"] == 3.5 and tm["restore_s"] == 0.25
    eng.release(1)
    assert ses.calls[-1] == ("release", 1)
    # failure reporting: empty while healthy, the device's message once a kernel has given up, and it sticks
    assert eng.failure() == ""
    ses.device_error = "device error word: code 1 detail 0x21000001"
    assert "code 1" in eng.failure()
    ses.device_error = ""
    assert "code 1" in eng.failure()


def test_open_failure_reports_the_reason(monkeypatch):
    from qwb200 import capi_impl
    from qwb200.native import build as nbuild
    from qwserve import engine as E

    def refuse(o, rank, world, port):
        raise ValueError("the configuration does not fit the GPU: weights 68.7 GB + slots 219.9 GB")
    monkeypatch.setattr(capi_impl, "build_ops", refuse)
    with pytest.raises(E.EngineError, match="does not fit the GPU"):
        E.Engine({"synthetic": "full"}, nbuild.ENGINE_LIB)
    with pytest.raises(E.EngineError, match="devices must list"):
        E.Engine({"devices": [0, 1, 2]}, nbuild.ENGINE_LIB)


def test_media_prompts_through_the_c_abi(monkeypatch):
    """qw_acquire_media / qw_begin_prompt with media descriptors: the structs are read through the shim, the pad tokens of
    the prompt reach the session as vision token ids, the same ids in every call of the request."""
    import numpy as np
    from qwb200 import capi_impl
    from qwb200.models.config import ModelConfig
    from qwb200.native import build as nbuild
    from qwb200.vision import VisionConfig
    from qwb200.vision.frontend import VisionFrontend
    from qwserve import engine as E

    class Enc:
        cfg = VisionConfig(depth=1, out_dim=ModelConfig.tiny().hidden)

        def encode(self, *a):
            raise AssertionError("the tower runs only when a slice is looked up")
    cfg, vc = ModelConfig.tiny(), Enc.cfg
    ses = ScriptedSession()
    monkeypatch.setattr(capi_impl, "build_ops", lambda o, r, w, p: capi_impl.SessionOps(ses, VisionFrontend(Enc(), 1 << 20)))
    eng = E.Engine({"synthetic": "tiny"}, nbuild.ENGINE_LIB)
    try:
        assert eng.has_vision is True
        h, w = 4, 6
        n_img = h * w // (vc.merge * vc.merge)
        patches = np.random.default_rng(2).standard_normal((2 * h * w, vc.patch_in)).astype(np.float32)
        starts = np.asarray([3], dtype=np.int64)
        toks = E.Tokens([5, 6, 7] + [cfg.image_pad] * n_img + [8, 9])
        m = E.Media(hash=99, video=0, t=1, h=h, w=w, patches=patches.ctypes.data, starts=starts.ctypes.data)
        assert eng.acquire(toks, 10, media=[m]) == 1
        got = ses.calls[-1][1]
        assert got[:3] == [5, 6, 7] and got[-2:] == [8, 9] and all(t < 0 for t in got[3:3 + n_img]) and len(set(got[3:3 + n_img])) == n_img
        assert eng.begin_prompt(1, toks, media=[m]) == 256 and ses.calls[-1][2] == got
        eng.prefetch(1, toks, media=[m])
        assert ses.calls[-1] == ("prefetch", got)
        # a media slice that lies outside the prompt is refused with a message, not a crash
        bad = np.asarray([len(toks)], dtype=np.int64)
        m2 = E.Media(hash=100, video=0, t=1, h=h, w=w, patches=patches.ctypes.data, starts=bad.ctypes.data)
        with pytest.raises(E.EngineError):
            eng.acquire(toks, 10, media=[m2])
    finally:
        eng.close()
