"""The speculative generation loop's host logic on CPU, over a fake engine whose "model" is a fixed next-token rule:
speculative output equals plain output whatever the drafts are, forced acceptance emits exactly 1 + a tokens, drafting
that never pays is switched off for growing stretches and its skipped MTP rows are caught up when it resumes, budgets,
stop tokens, the row limit of a step and the per-request run limit are respected."""
import types

import pytest
import torch

from qwb200.engine.engine import Slot
from qwb200.engine.sampling import SamplingParams
from qwb200.session import session as S

V = 97


def nxt(t):
    return (t * 7 + 3) % V


class FakeEngine:
    MAX_DRAFTS = 12

    def __init__(self, slots=2, wrong=lambda pos: False, max_rows=32, slot_tokens=4096):
        self.cfg = types.SimpleNamespace(vocab=V)
        self.opts = types.SimpleNamespace(slots=slots, max_rows=max_rows)
        self.dm = types.SimpleNamespace(max_rows=max_rows, slot_tokens=slot_tokens, buf={"gdn_save": None}, lib=None, dev="cpu",
                                        sc=types.SimpleNamespace(ranks=1))
        self.slot = [Slot() for _ in range(slots)]
        self.mtp = True
        self.wrong = wrong
        self.rows = None
        self.draft_calls, self.verify_rows, self.caught_up = 0, [], []

    def start(self, slot, prompt):
        self.slot[slot].tokens = list(prompt)
        self.slot[slot].mtp_hidden = torch.zeros(4)
        return nxt(prompt[-1])                       # the pending token: sampled from the prompt's last row, not fed yet

    def draft_batch(self, slots, pendings, k):
        self.draft_calls += 1
        out = []
        for s, p in zip(slots, pendings):
            cur, pos, d = p, self.slot[s].n, []
            for j in range(min(k, self.MAX_DRAFTS)):
                t = nxt(cur)
                if self.wrong(pos + j + 1):
                    t = (t + 1) % V
                d.append(t)
                cur = t
            out.append(d)
        return out

    def _logits(self, toks):
        rows = torch.full((len(toks), V), -10.0)
        for i, t in enumerate(toks):
            rows[i, nxt(t)] = 10.0
        return rows

    def verify_batch(self, slots, runs):
        flat = [t for r in runs for t in r]
        assert len(flat) <= self.dm.max_rows
        self.verify_rows.append([len(r) for r in runs])
        self.rows = self._logits(flat)
        return len(flat)

    def full_logits(self, n):
        return self.rows[:n]

    def accept_batch(self, slots, runs, n_acc):
        for s, run, na in zip(slots, runs, n_acc):
            self.slot[s].tokens.extend(run[:na])
            self.slot[s].mtp_hidden = torch.zeros(4)

    def mtp_catch_up(self, slot, rows):
        self.caught_up.append((slot, [(t, p) for _, t, p in rows]))


class FakeSampler:
    def __init__(self, *a, **kw):
        self.noted = []
        self.host_only = False

    def reset_slot(self, slot):
        pass

    def note_tokens(self, slot, tokens, generated):
        self.noted.append((slot, list(tokens)))

    def sample(self, logits, params, slots, positions, hists=None, force_host=None):
        assert logits.shape[0] == len(params) == len(slots) == len(positions)
        return [int(x) for x in logits.argmax(-1)], [0.0] * len(params)


class FakeIO:
    kv_block_bytes = 1024

    def __init__(self, dm):
        pass

    def state_layout_id(self):
        return 7


@pytest.fixture
def make(monkeypatch):
    monkeypatch.setattr(S, "GpuSampler", FakeSampler)
    monkeypatch.setattr(S, "StateIO", FakeIO)

    def build(**kw):
        eng = FakeEngine(**kw)
        return eng, S.Session(eng, host_cache_bytes=0)
    return build


def plain(first, n):
    out, t = [], first
    for _ in range(n):
        out.append(t)
        t = nxt(t)
    return out


def run(ses, eng, slot, pending, n_new, k, **kw):
    out = []
    while len(out) < n_new:
        o = ses.generate([S.StepReq(slot, pending, n_new - len(out), 0, SamplingParams())], k, **kw)[0]
        assert 1 <= len(o.tokens) <= k + 1
        out += o.tokens
        pending = o.tokens[-1]
    return out


@pytest.mark.parametrize("wrong", [lambda p: False, lambda p: p % 3 == 0, lambda p: True])
def test_speculative_output_equals_plain(make, wrong):
    eng, ses = make(wrong=wrong)
    pending = eng.start(0, [5, 6, 7])
    got = run(ses, eng, 0, pending, 60, k=4)
    # what a request emits are the tokens after its pending one; the pending token itself was emitted by the step before
    assert got == plain(nxt(pending), 60)
    assert eng.slot[0].tokens == [5, 6, 7] + plain(pending, 60)         # everything emitted but the newest token has been fed


def test_forced_acceptance_emits_exactly_one_plus_a(make):
    eng, ses = make(slots=4, wrong=lambda p: True)
    pend = [eng.start(s, [1, 2, 3 + s]) for s in range(4)]
    for a in range(6):
        outs = ses.generate([S.StepReq(s, pend[s], 64, 0, SamplingParams()) for s in range(4)], 5, force_accept=a)
        assert [len(o.tokens) for o in outs] == [1 + a] * 4
        assert [o.first_row for o in outs] == [i * (1 + a) for i in range(4)]
        assert eng.verify_rows[-1] == [6] * 4                             # one step verifies all four runs
        pend = [o.tokens[-1] for o in outs]


def test_drafting_that_never_pays_pauses_and_catches_up(make):
    eng, ses = make(wrong=lambda p: True)
    pending = eng.start(0, [9, 8, 7])
    si = ses.slots[0]
    steps_with_drafts = steps_plain = 0
    stretches = []
    for _ in range(400):
        before = eng.draft_calls
        was_plain = si.plain_left > 0
        o = ses.generate([S.StepReq(0, pending, 1000, 0, SamplingParams())], 4)[0]
        pending = o.tokens[-1]
        if eng.draft_calls > before:
            steps_with_drafts += 1
        else:
            steps_plain += 1
        if si.plain_left > 0 and not was_plain:
            stretches.append(si.plain_left)
    # the acceptance average falls until drafting stops paying; stretches grow 32 -> 80 -> 128 -> 176 (each counted after its first step)
    assert steps_plain > 300 and 0 < steps_with_drafts < 60
    assert stretches[:4] == [31, 79, 127, 175]
    # every row skipped during a stretch was handed to the MTP layer when drafting resumed, in position order, none twice
    caught = [p for _, rows in eng.caught_up for _, p in rows]
    assert caught == sorted(set(caught)) and len(caught) >= 32 + 80
    assert ses.catch_up_rows == len(caught)
    assert eng.slot[0].tokens[3:] == plain(nxt([9, 8, 7][-1]), len(eng.slot[0].tokens) - 3)


def test_budget_stop_token_and_limits(make, capsys):
    eng, ses = make(slots=8, max_rows=32)
    pend = [eng.start(s, [11, 12, 13 + s]) for s in range(8)]
    # budget: at most budget tokens come back, and no more drafts than budget - 1 are made
    o = ses.generate([S.StepReq(0, pend[0], 2, 0, SamplingParams())], 6)[0]
    assert len(o.tokens) == 2 and eng.verify_rows[-1] == [2]
    with pytest.raises(ValueError):
        ses.generate([S.StepReq(0, o.tokens[-1], 0, 0, SamplingParams())], 6)
    # a stop token ends the run where it is sampled, whatever drafts follow
    p1 = pend[1]
    stop_at = plain(nxt(p1), 3)[2]
    ses.set_stop_tokens(1, [stop_at])
    got, o = [], None
    while o is None or not o.stopped:
        o = ses.generate([S.StepReq(1, p1 if not got else got[-1], 64, 0, SamplingParams())], 6)[0]
        got += o.tokens
    assert got == plain(nxt(p1), 3) and o.tokens[-1] == stop_at          # nothing after the stop token, although drafts went past it
    # eight requests asking for 12 drafts each do not fit 32 rows: the longest runs are trimmed, every request keeps its row
    for si in ses.slots:
        si.accept = 0.99                                                  # drafting pays: the longest run allowed is asked for
    reqs = [S.StepReq(s, pend[s], 64, 0, SamplingParams()) for s in range(2, 8)]
    ses.generate(reqs, 12)
    assert sum(eng.verify_rows[-1]) <= 32 and min(eng.verify_rows[-1]) >= 5 and len(eng.verify_rows[-1]) == 6
    # the per-request run limit and the acceptance log
    ses.spec_max_rows, ses.spec_log = 3, True
    capsys.readouterr()
    o = ses.generate([S.StepReq(0, nxt(eng.slot[0].tokens[-1]), 64, 0, SamplingParams())], 12)[0]
    assert eng.verify_rows[-1] == [3] and len(o.tokens) == 3
    assert "spec: slot 0" in capsys.readouterr().out
    # a slot with no room left for the run
    eng.dm.slot_tokens = eng.slot[0].n + 2
    o = ses.generate([S.StepReq(0, o.tokens[-1], 64, 0, SamplingParams())], 12)[0]
    assert eng.verify_rows[-1] == [2]
    eng.dm.slot_tokens = eng.slot[0].n
    with pytest.raises(ValueError, match="full"):
        ses.generate([S.StepReq(0, o.tokens[-1], 64, 0, SamplingParams())], 12)
