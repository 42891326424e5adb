"""Sampled generation with the real host sampler over the rule-based engine: a token drawn at a position depends on the
seed and the history up to there only, so speculative decoding (greedy drafts, most of them rejected by the draw) must
give the tokens of plain decoding, with and without penalties - the property that makes speculation exact."""
import pytest

from rule_engine import HostRowSampler, RuleEngine, RuleIO


def run(monkeypatch, k, sp, n_new, prompt):
    from qwb200.session import session as S
    monkeypatch.setattr(S, "GpuSampler", HostRowSampler)
    monkeypatch.setattr(S, "StateIO", RuleIO)
    eng = RuleEngine(vocab=300, modulus=256, slots=1)
    eng.spread = True
    ses = S.Session(eng, host_cache_bytes=0)
    ses.io.e = eng
    slot = ses.acquire(prompt, n_new)
    ses.begin_prompt(slot, prompt)
    while not ses.prefill_some(slot, 4096):
        pass
    tok, lp = ses.sample_prompt(slot, sp)
    out, lps = [tok], [lp]
    ses.slots[slot].accept = 0.9                         # keep drafting although most drafts will be rejected
    while len(out) < n_new:
        o = ses.generate([S.StepReq(slot, out[-1], n_new - len(out), 0, sp)], k)[0]
        out += o.tokens
        lps += o.logprobs
        ses.slots[slot].accept = 0.9
    return out, lps, eng


@pytest.mark.parametrize("params", [dict(temperature=1.0, top_k=20, top_p=0.95, seed=1234),
                                    dict(temperature=1.3, min_p=0.05, seed=99),
                                    dict(temperature=1.0, top_k=4, presence_penalty=1.5, repetition_penalty=1.1, frequency_penalty=0.2, seed=7)])
def test_sampled_speculation_equals_sampled_plain_decoding(monkeypatch, params):
    from qwb200.engine.sampling import SamplingParams
    sp = SamplingParams(**params)
    prompt = [(i * 11) % 250 for i in range(40)]
    plain, lp0, _ = run(monkeypatch, 0, sp, 48, prompt)
    spec, lp1, eng = run(monkeypatch, 4, sp, 48, prompt)
    assert spec == plain and max(abs(a - b) for a, b in zip(lp0, lp1)) < 1e-6
    assert eng.draft_calls > 5 and len(set(plain)) > 8               # drafts ran, and the draw really wandered off the greedy path
    greedy = []
    t = prompt[-1]
    for _ in range(48):
        t = eng.nxt(t)
        greedy.append(t)
    assert plain != greedy
