"""GPU sampler against the native host sampler: greedy, penalties, truncation, frequencies, seeds."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(V=5000, slots=2):
    from qwb200.engine.sampling import GpuSampler
    from qwb200.ops import lib as qlib
    return GpuSampler(qlib.load(required=True), "cuda:0", V, slots, 32, seed=3)


def test_greedy_and_penalties_match_host():
    from qwb200.engine.sampling import SamplingParams
    from qwb200.native import host as H
    s = make()
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn(4, 5000, generator=g, device="cuda") * 3
    hist = [int(torch.argmax(logits[0])), 17, 17, 900]
    s.note_tokens(0, hist[:2], generated=False)
    s.note_tokens(0, hist[2:], generated=True)
    P = [SamplingParams(), SamplingParams(repetition_penalty=1.7), SamplingParams(presence_penalty=5.0, frequency_penalty=1.0),
         SamplingParams(temperature=0.0, repetition_penalty=1.3, presence_penalty=0.4)]
    toks, lps = s.sample(logits[:1].expand(4, -1).contiguous(), P, [0, 0, 0, 0], [4] * 4)
    host = H.HostSampler(0)
    for i, p in enumerate(P):
        t, lp = host.sample(logits[0].cpu().numpy(), p.to_host(), hist, 2)
        assert toks[i] == t and abs(lps[i] - lp) < 1e-3


def test_truncated_draws_stay_in_the_host_set_and_follow_the_distribution():
    from qwb200.engine.sampling import SamplingParams
    s = make(V=3000)
    logits = torch.full((1, 3000), -20.0, device="cuda")
    logits[0, [5, 70, 900, 2999]] = torch.tensor([2.0, 1.5, 1.0, 0.0], device="cuda")
    n = 3000
    rows = logits.expand(32, -1).contiguous()
    def freq(p):
        c = {}
        for rep in range(n // 32):
            toks, _ = s.sample(rows, [p] * 32, [0] * 32, list(range(rep * 32, rep * 32 + 32)))
            for t in toks:
                c[t] = c.get(t, 0) + 1
        return {k: v / (n // 32 * 32) for k, v in c.items()}
    f = freq(SamplingParams(temperature=1.0, top_k=2))
    assert set(f) == {5, 70} and abs(f[5] - 1 / (1 + np.exp(-0.5))) < 0.04
    f = freq(SamplingParams(temperature=1.0, top_p=0.8))
    w = np.exp([2.0, 1.5, 1.0, 0.0]); w /= w.sum() + 2996 * np.exp(-20.0)
    assert set(f) == {5, 70, 900}                      # smallest prefix reaching 0.8 of the mass
    assert abs(f[5] - w[0] / w[:3].sum()) < 0.04
    f = freq(SamplingParams(temperature=1.0, min_p=0.5))
    assert set(f) == {5, 70}                           # weights >= half of the best token's
    f = freq(SamplingParams(temperature=1.0))          # untruncated: Gumbel-max over the vocabulary
    assert abs(f[5] - w[0]) < 0.04 and abs(f.get(2999, 0) - w[3]) < 0.03
    f = freq(SamplingParams(temperature=0.5, top_k=3))
    w2 = np.exp(np.array([2.0, 1.5, 1.0]) / 0.5); w2 /= w2.sum()
    assert abs(f[5] - w2[0]) < 0.04


def test_seed_and_position_fix_the_draw_and_wide_nucleus_falls_back():
    from qwb200.engine.sampling import SamplingParams
    s = make(V=4000)
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(8, 4000, generator=g, device="cuda")
    p = SamplingParams(temperature=1.0, top_k=50, seed=1234)
    a, _ = s.sample(logits, [p] * 8, [0] * 8, [10] * 8)
    b, _ = s.sample(logits, [p] * 8, [0] * 8, [10] * 8)
    c, _ = s.sample(logits, [p] * 8, [0] * 8, [11] * 8)
    assert a == b and a != c
    # a flat distribution with top_p = 0.99 needs far more than 256 candidates: the host finishes the row
    flat = torch.zeros(1, 4000, device="cuda")
    before = s.fallbacks
    t, lp = s.sample(flat, [SamplingParams(temperature=1.0, top_p=0.99)], [0], [0], hists=[((), 0)])
    assert s.fallbacks == before + 1 and 0 <= t[0] < 4000 and abs(lp[0] + np.log(4000)) < 1e-3
