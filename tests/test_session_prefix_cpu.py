"""The session's prompt life cycle on CPU over a fake engine whose state is a pure function of the tokens it was fed
(KV rows = the tokens, recurrent state = a running checksum): whatever way a prompt starts - from nothing, continuing
what the slot holds, from a device snapshot at a message boundary, from the block store - the state after its prefill
must equal the state of feeding the whole prompt from scratch, and the reuse counters must say what was skipped."""
import types

import numpy as np
import pytest
import torch

from qwb200.engine.engine import Slot
from qwb200.session import session as S

V, BLOCK, BOUNDARY = 1000, 256, 999


def checksum(state: int, toks) -> int:
    for t in toks:
        state = (state * 1000003 + int(t) + 1) % (1 << 61)
    return state


class FakeEngine:
    MAX_DRAFTS = 12

    def __init__(self, slots=3, cap=8192):
        self.cfg = types.SimpleNamespace(vocab=V)
        self.opts = types.SimpleNamespace(slots=slots, max_rows=32)
        self.dm = types.SimpleNamespace(max_rows=32, slot_tokens=cap, buf={}, lib=None, dev="cpu", sc=types.SimpleNamespace(ranks=1))
        self.slot = [Slot() for _ in range(slots)]
        self.kv = [np.full(cap, -1, np.int32) for _ in range(slots)]      # "KV row" of position p: the token fed there
        self.state = [0] * slots                                           # "recurrent state": checksum of everything fed
        self.mtp = False
        self.fed = 0
        self.last_prefill_row = 0

    def reset(self, slot):
        self.slot[slot].tokens = []
        self.slot[slot].mtp_hidden = None
        self.kv[slot][:] = -1
        self.state[slot] = 0

    def prefill(self, slot, piece, want_logits=True):
        sl = self.slot[slot]
        self.kv[slot][sl.n:sl.n + len(piece)] = piece
        self.state[slot] = checksum(self.state[slot], piece)
        sl.tokens.extend(piece)
        self.fed += len(piece)
        self.last_prefill_row = 0

    def full_logits(self, n):
        return torch.zeros(n, V)

    def consistent(self, slot, toks):
        n = len(toks)
        return (self.slot[slot].tokens == list(toks) and self.state[slot] == checksum(0, toks)
                and np.array_equal(self.kv[slot][:n], np.asarray(toks, np.int32)))


class FakeIO:
    MAX_BATCH = 8
    kv_block_bytes = BLOCK * 4

    def __init__(self, dm):
        self.e = None          # set by the fixture

    def state_layout_id(self):
        return 42

    def recurrent_bytes(self):
        return 8

    def export_kv(self, slot, bi):
        return self.e.kv[slot][bi * BLOCK:(bi + 1) * BLOCK].tobytes()

    def import_kv(self, slot, bi, payload):
        self.e.kv[slot][bi * BLOCK:(bi + 1) * BLOCK] = np.frombuffer(payload, np.int32)

    def export_recurrent(self, slot):
        return int(self.e.state[slot]).to_bytes(8, "little")

    def import_recurrent(self, slot, payload):
        self.e.state[slot] = int.from_bytes(payload, "little")

    def snapshot_save(self, slot):
        return [torch.tensor([self.e.state[slot]], dtype=torch.int64)]

    def snapshot_restore(self, slot, tensors):
        self.e.state[slot] = int(tensors[0][0])


class FakeSampler:
    def __init__(self, *a, **kw):
        self.host_only = False
        self.counts = {}

    def reset_slot(self, slot):
        self.counts[slot] = [0, 0]

    def note_tokens(self, slot, tokens, generated):
        self.counts.setdefault(slot, [0, 0])[1 if generated else 0] += len(tokens)

    def sample(self, logits, params, slots, positions, hists=None, force_host=None):
        return [1] * len(params), [0.0] * len(params)


@pytest.fixture
def ses(monkeypatch):
    monkeypatch.setattr(S, "GpuSampler", FakeSampler)
    monkeypatch.setattr(S, "StateIO", FakeIO)
    eng = FakeEngine()
    s = S.Session(eng, host_cache_bytes=64 << 20, prefill_piece=512)
    s.io.e = eng
    s.set_boundary_token(BOUNDARY)
    return s


def message(seed, n):
    """n - 1 ordinary tokens and the end-of-message token."""
    g = np.random.default_rng(seed)
    return [int(x) for x in g.integers(1, 900, n - 1)] + [BOUNDARY]


def fill(ses, slot, prompt, piece=512):
    reused = ses.begin_prompt(slot, prompt)
    steps = 0
    while not ses.prefill_some(slot, piece):
        steps += 1
        assert steps < 100
    assert ses.e.consistent(slot, prompt), "the slot's state is not that of the prompt fed from scratch"
    return reused


def test_every_way_to_start_a_prompt_gives_the_same_state(ses):
    eng = ses.e
    system, user1 = message(1, 1300), message(2, 700)
    p1 = system + user1
    # ---- from nothing, in pieces that end on block boundaries
    slot = ses.acquire(p1, 100)
    assert slot == 0 and fill(ses, slot, p1) == 0
    assert eng.fed == len(p1) and len(ses.slots[0].block_keys) == len(p1) // BLOCK
    st = ses.cache_stats()
    assert st["prompt_tokens"] == len(p1) and st["reused_tokens"] == 0 and st["blocks"] == len(p1) // BLOCK and st["snapshots"] >= 1
    # ---- the next turn continues in place: only the new tokens are fed
    answer, user2 = message(3, 200), message(4, 300)
    eng.prefill(0, answer)                                   # what generation appended to the slot
    ses.release(0)
    p2 = p1 + answer + user2
    assert ses.acquire(p2, 100) == 0                          # the slot that holds the most of it
    fed0 = eng.fed
    assert fill(ses, 0, p2) == len(p1) + len(answer) and eng.fed - fed0 == len(user2)
    ses.release(0)
    # ---- an edited last message: back to the device snapshot taken at the message boundary before it
    p3 = p1 + answer + message(5, 260)
    assert ses.acquire(p3, 100) == 0
    fed0 = eng.fed
    reused = fill(ses, 0, p3)
    assert reused == len(p1)                                  # the snapshot taken when the first turn's prompt was in (its end is a boundary)
    assert eng.fed - fed0 == len(p3) - reused
    # ---- another slot, the same system prompt, a different user: the block store serves the stored prefix
    ses.slots[0].busy = True
    p4 = system + message(6, 500)
    slot = ses.acquire(p4, 100)
    assert slot == 1
    fed0 = eng.fed
    reused = fill(ses, 1, p4)
    assert reused >= 1024 and reused % BLOCK == 0 and reused <= len(system) and eng.fed - fed0 == len(p4) - reused
    assert ses.cache_stats()["hits"] >= 1 and ses.slots[1].timing["restore_s"] > 0
    # ---- nothing in common: a reset
    p5 = message(7, 400)
    ses.release(1)
    ses.slots[1].busy = True
    slot = ses.acquire(p5, 10)
    assert slot == 2 and fill(ses, 2, p5) == 0
    st = ses.cache_stats()
    assert st["prompt_tokens"] == sum(map(len, (p1, p2, p3, p4, p5))) and st["reused_tokens"] > len(p1)
    assert st["blend_candidate_tokens"] > 0                   # chunks seen before at another position or after another prefix


def test_persist_thinning_and_no_store(ses, monkeypatch):
    eng = ses.e
    p = message(11, 1536)
    ses.acquire(p, 10)
    ses.snap_keep_gap = 600                                   # QW_SNAP_KEEP_GAP: stored snapshots closer than this to the next are dropped
    fill(ses, 0, p, piece=256)                                # a snapshot would be stored after every block
    st = ses.cache_stats()
    assert st["blocks"] == 6 and 1 <= st["snapshots"] <= 3
    ses.persist()
    # a stored prefix is found again by a fresh slot even after the first one was reset
    eng.reset(0)
    ses.release(0)
    ses.slots[0].busy = True
    q = p + message(12, 100)
    slot = ses.acquire(q, 10)
    assert fill(ses, slot, q) == 1536
    # without a store tier nothing is exported
    s2 = S.Session(eng, host_cache_bytes=0)
    s2.io.e = eng
    assert not s2.store_on and s2.pool is None
    eng.reset(2)
    s2.slots[2].busy = True
    s2.begin_prompt(2, p)
    while not s2.prefill_some(2, 512):
        pass
    assert s2.cache_stats()["blocks"] == 0 and s2.slots[2].block_keys == []


def test_common_prefix_blocks():
    import random
    rnd = random.Random(4)
    for n, m in ((0, 5), (5, 0), (1, 1), (4095, 4096), (4096, 4096), (10000, 9000), (20000, 20000)):
        a = [rnd.randrange(50) for _ in range(n)]
        for cut in {0, 1, min(n, m) // 2, max(0, min(n, m) - 1), min(n, m)}:
            b = a[:cut] + [99] * (m - cut) if cut < m else a[:m]
            want = 0
            while want < min(len(a), len(b)) and a[want] == b[want]:
                want += 1
            assert S.common_prefix(a, b) == want and S.common_prefix(tuple(a), b, block=7) == want
