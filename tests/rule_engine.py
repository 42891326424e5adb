"""A stand-in for ``Engine`` that needs no device: its "model" is a fixed next-token rule, its "KV rows" are the tokens it
was fed and its "recurrent state" a checksum of them.  It has the whole interface the session uses - prefill, decode,
drafts, verification, acceptance, state export / import - so the real ``Session`` (native planner, block store, chunker)
runs over it on CPU, alone or behind the C ABI and the server.  Drafts are wrong where ``wrong(position)`` says so."""
import types

import numpy as np
import torch

from qwb200.engine.engine import Slot

BLOCK = 256


def checksum(state: int, toks) -> int:
    for t in toks:
        state = (state * 1000003 + int(t) + 1) % (1 << 61)
    return state


class RuleEngine:
    MAX_DRAFTS = 12

    def __init__(self, vocab=512, slots=3, cap=8192, max_rows=32, mtp=True, wrong=lambda pos: False, stop_after=None, stop_token=None, modulus=None):
        self.V = vocab
        self.modulus = modulus or vocab          # the rule's tokens stay below this (e.g. inside a tokenizer's byte range)
        self.cfg = types.SimpleNamespace(vocab=vocab)
        self.opts = types.SimpleNamespace(slots=slots, max_rows=max_rows)
        self.dm = types.SimpleNamespace(max_rows=max_rows, slot_tokens=cap, buf={"gdn_save": None}, lib=None, dev="cpu",
                                        sc=types.SimpleNamespace(ranks=1), check_error=lambda: None)
        self.slot = [Slot() for _ in range(slots)]
        self.kv = [np.full(cap, -1, np.int32) for _ in range(slots)]
        self.state = [0] * slots
        self.mtp = mtp
        self.wrong = wrong
        self.stop_after, self.stop_token = stop_after, stop_token       # the rule emits stop_token after that many tokens of a sequence
        self.rows = None
        self.last_prefill_row = 0
        self.fed = self.draft_calls = 0
        self.verify_rows, self.caught_up = [], []

    # ---- the model
    def nxt(self, t, pos=None):
        if self.stop_after is not None and pos is not None and pos >= self.stop_after:
            return self.stop_token
        return (int(t) * 7 + 3) % self.modulus

    def _logits(self, toks, positions):
        rows = torch.full((len(toks), self.V), -10.0)
        for i, (t, p) in enumerate(zip(toks, positions)):
            top = self.nxt(t, p)
            rows[i, top] = 10.0
            if getattr(self, "spread", False):          # a distribution worth sampling from: four close candidates
                for j, v in enumerate((9.6, 9.3, 8.9)):
                    rows[i, (top + 17 * (j + 1)) % self.modulus] = v
        return rows

    # ---- what the session calls
    def reset(self, slot):
        self.slot[slot].tokens = []
        self.slot[slot].mtp_hidden = None
        self.kv[slot][:] = -1
        self.state[slot] = 0

    def _feed(self, slot, toks):
        sl = self.slot[slot]
        self.kv[slot][sl.n:sl.n + len(toks)] = toks
        self.state[slot] = checksum(self.state[slot], toks)
        sl.tokens.extend(int(t) for t in toks)
        self.fed += len(toks)
        if self.mtp:
            sl.mtp_hidden = torch.zeros(4)

    def prefill(self, slot, piece, want_logits=True):
        base = self.slot[slot].n
        self._feed(slot, piece)
        self.rows = self._logits(piece[-1:], [base + len(piece) - 1])
        self.last_prefill_row = 0
        return self.rows[0]

    def decode(self, slots, tokens, flags=0, sync=True):
        pos = [self.slot[s].n for s in slots]
        for s, t in zip(slots, tokens):
            self._feed(s, [t])
        self.rows = self._logits(tokens, pos)
        return [int(x) for x in self.rows.argmax(-1)]

    def full_logits(self, n):
        return self.rows[:n]

    def draft_batch(self, slots, pendings, k):
        self.draft_calls += 1
        out = []
        for s, p in zip(slots, pendings):
            cur, pos, d = p, self.slot[s].n, []
            for j in range(min(k, self.MAX_DRAFTS)):
                t = self.nxt(cur, pos + j)
                if self.wrong(pos + j + 1):
                    t = (t + 1) % self.modulus
                d.append(t)
                cur = t
            out.append(d)
        return out

    def verify_batch(self, slots, runs):
        flat, pos = [], []
        for s, run in zip(slots, runs):
            flat += list(run)
            pos += list(range(self.slot[s].n, self.slot[s].n + len(run)))
        assert len(flat) <= self.dm.max_rows
        self.verify_rows.append([len(r) for r in runs])
        self.rows = self._logits(flat, pos)
        return len(flat)

    def accept_batch(self, slots, runs, n_acc):
        self.accepts = getattr(self, "accepts", 0) + 1
        for i, (s, run, na) in enumerate(zip(slots, runs, n_acc)):
            self._feed(s, run[:na])
            if self.accepts == getattr(self, "fail_accept_at", -1) and i == 0:
                raise RuntimeError("injected: the accept launch failed after the first request's rows were kept")

    def mtp_catch_up(self, slot, rows):
        self.caught_up.append((slot, [(t, p) for _, t, p in rows]))

    def consistent(self, slot, toks):
        n = len(toks)
        return (self.slot[slot].tokens == [int(t) for t in toks] and self.state[slot] == checksum(0, toks)
                and np.array_equal(self.kv[slot][:n], np.asarray(toks, np.int32)))


class RuleIO:
    """``StateIO`` over a RuleEngine: a KV block is the block's tokens, the recurrent state its checksum."""
    MAX_BATCH = 8
    kv_block_bytes = BLOCK * 4

    def __init__(self, dm):
        self.e = None          # the engine; set by ``install``

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


class ArgmaxSampler:
    """``GpuSampler``'s interface with a greedy draw on the host."""

    def __init__(self, *a, **kw):
        self.host_only = False

    def reset_slot(self, slot):
        pass

    def note_tokens(self, slot, tokens, generated):
        pass

    def sample(self, logits, params, slots, positions, hists=None, force_host=None):
        assert logits.shape[0] == len(params) == len(slots) == len(positions)
        lse = torch.logsumexp(logits.float(), -1)
        top = logits.argmax(-1)
        return [int(x) for x in top], [float(logits[i, top[i]] - lse[i]) for i in range(len(params))]


def make_session(monkeypatch, engine, **kw):
    """A real Session over ``engine`` (block store and planner native, sampler and state I/O replaced)."""
    from qwb200.session import session as S
    monkeypatch.setattr(S, "GpuSampler", ArgmaxSampler)
    monkeypatch.setattr(S, "StateIO", RuleIO)
    ses = S.Session(engine, **kw)
    ses.io.e = engine
    return ses


class RuleOps:
    """A rank's ``SessionOps`` over a real Session on a RuleEngine, plus ``dump`` (what the rank holds, for comparing
    ranks).  ``build_rank`` is the ``--builder`` of worker processes."""

    def __new__(cls, o, patch_module=False):
        from qwb200 import capi_impl
        from qwb200.session import session as S
        if patch_module:          # a worker process of its own; in the test process the caller patches (and restores) the module
            S.GpuSampler, S.StateIO = ArgmaxSampler, RuleIO
        assert S.GpuSampler is ArgmaxSampler and S.StateIO is RuleIO, "patch qwb200.session.session first"
        wrong = (lambda p: p % 3 == 0) if o.get("unreliable_drafts") else (lambda p: False)
        eng = RuleEngine(vocab=512, modulus=256, slots=int(o.get("slots", 3)), wrong=wrong)
        ses = S.Session(eng, host_cache_bytes=8 << 20)
        ses.io.e = eng

        class Ops(capi_impl.SessionOps):
            def dump(self, path):
                import json
                with open(f"{path}.rank{o.get('rank', 0)}", "w") as f:
                    json.dump({"tokens": [sl.tokens for sl in eng.slot], "state": eng.state, "fed": eng.fed,
                               "stats": {k: int(v) for k, v in ses.cache_stats().items()}}, f)
                return 0
        return Ops(ses, None)


def build_rank(open_message, world, patch_module=True):
    return RuleOps(dict(open_message.get("options", {}), rank=open_message.get("rank", 0)), patch_module=patch_module)


def patch_session_module(monkeypatch):
    from qwb200.session import session as S
    monkeypatch.setattr(S, "GpuSampler", ArgmaxSampler)
    monkeypatch.setattr(S, "StateIO", RuleIO)


class StubTower:
    """Stands where the vision encoder stands: the front end needs its geometry until a slice is looked up."""

    def __init__(self, hidden=64):
        from qwb200.vision import VisionConfig
        self.cfg = VisionConfig(depth=1, out_dim=hidden)

    def encode(self, *a):
        raise AssertionError("the tower runs only when a slice is looked up")


def build_rank_with_vision(open_message, world, patch_module=True):
    from qwb200.vision.frontend import VisionFrontend
    ops = build_rank(open_message, world, patch_module)
    ops.vision = VisionFrontend(StubTower(), 1 << 20)
    return ops


class HostRowSampler:
    """``GpuSampler``'s interface over the native host sampler: every row is drawn on the host from its history, which
    is what the engine does for rows the GPU sampler hands back."""

    def __init__(self, *a, **kw):
        from qwb200.native import host as H
        self.host = H.HostSampler(kw.get("seed", 0) if kw else 0)
        self.host_only = True

    def reset_slot(self, slot):
        pass

    def note_tokens(self, slot, tokens, generated):
        pass

    def sample(self, logits, params, slots, positions, hists=None, force_host=None):
        toks, lps = [], []
        for i, p in enumerate(params):
            hist, pend = hists[i]
            t, lp = self.host.sample(logits[i].float().numpy(), p.to_host(), list(hist), pend)
            toks.append(int(t))
            lps.append(float(lp))
        return toks, lps
