"""Randomised conversations against the real Session over the rule-based engine: new conversations, follow-up turns,
edited last messages, exact repeats, slots under pressure, random prefill pieces, unreliable drafts, snapshot thinning.
Invariants after every prompt: the slot's state is the state of the prompt fed from scratch, reuse never exceeds what
the prompt shares with something seen before, and what is generated is what the rule dictates."""
import random

import pytest

from rule_engine import RuleEngine, make_session

BOUNDARY = 999


def message(rnd, n):
    return [rnd.randrange(1, 900) for _ in range(n - 1)] + [BOUNDARY]


@pytest.mark.parametrize("seed", range(12))
def test_random_conversations_keep_every_invariant(monkeypatch, tmp_path, seed):
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    rnd = random.Random(seed)
    pattern = rnd.randrange(2, 9)
    eng = RuleEngine(vocab=1000, slots=3, cap=6144, wrong=lambda p: (p * 2654435761 >> 3) % pattern == 0)
    disk = dict(disk_cache_dir=str(tmp_path), disk_cache_bytes=64 << 20) if seed % 3 == 2 else {}      # some runs with a disk tier under a tiny RAM tier
    ram = (96 << 10) if (seed % 4 == 0 or disk) else (64 << 20)
    ses = make_session(monkeypatch, eng, host_cache_bytes=ram, prefill_piece=rnd.choice([256, 512, 1024]), **disk)
    ses.set_boundary_token(BOUNDARY)
    ses.snap_min_gap = rnd.choice([256, 512, 1024])
    ses.snap_keep_gap = rnd.choice([0, 0, 600])
    system = message(rnd, rnd.randrange(300, 1500))
    seen = []                       # every prompt fed so far, with what was generated after it
    held = []                       # slots kept busy for a while
    for step in range(30):
        kind = rnd.choice(["new", "new_sys", "follow", "edit", "repeat"]) if seen else "new_sys"
        if kind == "new":
            prompt = message(rnd, rnd.randrange(5, 700))
        elif kind == "new_sys":
            prompt = system + message(rnd, rnd.randrange(5, 400))
        else:
            base, gen = rnd.choice(seen)
            if kind == "follow":
                prompt = base + gen + message(rnd, rnd.randrange(5, 300))
            elif kind == "edit":
                cut = max(i for i, t in enumerate(base[:-1]) if t == BOUNDARY) + 1 if BOUNDARY in base[:-1] else 0
                prompt = base[:cut] + message(rnd, rnd.randrange(5, 300))
            else:
                prompt = list(base)
        if len(prompt) > 5000:
            continue
        n_new = rnd.randrange(1, 40)
        slot = ses.acquire(prompt, n_new)
        while slot < 0:
            assert held, "no slot although none is held"
            ses.release(held.pop(rnd.randrange(len(held))))
            slot = ses.acquire(prompt, n_new)
        if disk and rnd.random() < 0.5:                              # read-ahead of stored blocks that are only on disk
            ses.prefetch(prompt)
            import time
            t0 = time.time()
            while ses.loads_pending() and time.time() - t0 < 5:
                time.sleep(0.002)
        reused = ses.begin_prompt(slot, prompt)
        shared = max([0] + [next((i for i, (a, b) in enumerate(zip(prompt, p + g)) if a != b), min(len(prompt), len(p + g))) for p, g in seen])
        assert 0 <= reused <= min(shared, len(prompt)) and (reused < len(prompt) or prompt in [p for p, _ in seen])
        guard = 0
        while not ses.prefill_some(slot, rnd.choice([64, 256, 512, 4096])):
            guard += 1
            assert guard < 200
        assert eng.consistent(slot, prompt), (seed, step, kind)
        pending, _ = ses.sample_prompt(slot, SamplingParams())
        assert pending == eng.nxt(prompt[-1])
        out = [pending]
        k = rnd.choice([0, 1, 3, 6])
        while len(out) < n_new:
            o = ses.generate([StepReq(slot, out[-1], n_new - len(out), 0, SamplingParams())], k)[0]
            assert 1 <= len(o.tokens) <= k + 1
            out += o.tokens
        want, t = [], prompt[-1]
        for _ in range(len(out)):
            t = eng.nxt(t)
            want.append(t)
        assert out == want, (seed, step, kind)
        assert eng.consistent(slot, prompt + out[:-1])               # everything emitted but the newest token has been fed
        seen.append((prompt, out[:-1]))
        if rnd.random() < 0.4 and len(held) < 2:
            held.append(slot)
        else:
            ses.release(slot)
    ses.persist()
    st = ses.cache_stats()
    if disk:
        assert st["disk_bytes"] > 0
    assert st["prompt_tokens"] == sum(len(p) for p, _ in seen) and st["reused_tokens"] <= st["prompt_tokens"]
