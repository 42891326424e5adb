"""Session: prefix-cache restore equals recompute, slot choice, sampling entry points, speculative generate."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(tmp_path=None, slots=2, **kw):
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    from qwb200.session.session import Session
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=21)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=21)
    eng = Engine.from_weights(cfg, w, table, EngineOptions(slots=slots, slot_tokens=1024, use_graphs=False, save_gdn=True, **kw))
    return cfg, eng, Session(eng, host_cache_bytes=1 << 28, disk_cache_dir=str(tmp_path) if tmp_path else None,
                             disk_cache_bytes=1 << 30, prefill_piece=256)


def prompt_of(cfg, n, seed):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_restore_from_store_equals_recompute_and_slot_choice(tmp_path):
    from qwb200.engine.sampling import SamplingParams
    cfg, eng, ses = make(tmp_path)
    shared = prompt_of(cfg, 600, 1)
    a = shared + prompt_of(cfg, 50, 2)
    s0 = ses.acquire(a, 16)
    assert s0 == 0 and ses.begin_prompt(s0, a) == 0
    while not ses.prefill_some(s0, 256):
        pass
    la = ses.slots[s0].logits.clone()
    ta, _ = ses.sample_prompt(s0, SamplingParams())
    st = ses.cache_stats()
    assert st["blocks"] == 2 and st["snapshots"] >= 2
    # a second request sharing the 600-token prefix goes to the free slot and restores 512 tokens from the store
    b = shared + prompt_of(cfg, 40, 3)
    s1 = ses.acquire(b, 16)
    assert s1 == 1
    assert ses.begin_prompt(s1, b) == 512
    while not ses.prefill_some(s1, 1024):
        pass
    lb = ses.slots[s1].logits.clone()
    # recompute b from scratch on a fresh engine: same logits as after the restore
    cfg2, eng2, ses2 = make(None, slots=1)
    s = ses2.acquire(b, 16)
    assert ses2.begin_prompt(s, b) == 0
    while not ses2.prefill_some(s, 1024):
        pass
    ref = ses2.slots[s].logits
    assert float((lb - ref).abs().max() / ref.abs().max()) < 2e-2
    assert int(torch.argmax(lb)) == int(torch.argmax(ref))
    # follow-up turn on slot 0: everything it holds is kept
    ses.release(s0)
    a2 = a + [ta] + prompt_of(cfg, 20, 4)
    ses.e.decode([s0], [ta])                                  # the sampled token joins the slot
    assert ses.acquire(a2, 8) == s0 and ses.begin_prompt(s0, a2) == len(a) + 1
    ses.persist()
    assert ses.cache_stats()["disk_bytes"] > 0 and ses.cache_stats()["hits"] == 1


def test_generate_greedy_matches_engine_and_sampling_runs():
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    cfg, eng, ses = make(None, slots=2)
    p = prompt_of(cfg, 80, 5)
    s = ses.acquire(p, 64)
    ses.begin_prompt(s, p)
    while not ses.prefill_some(s, 4096):
        pass
    first, lp = ses.sample_prompt(s, SamplingParams())
    assert lp <= 0
    # reference continuation on a second engine
    cfg2, eng2, ses2 = make(None, slots=1)
    eng2.prefill(0, p)
    want = eng2.generate_greedy(0, first, 20, k=0)
    ses.set_stop_tokens(s, [])
    got, pending = [], first
    while len(got) < 20:
        out = ses.generate([StepReq(s, pending, 20 - len(got), 0, SamplingParams())], k=3)[0]
        assert 1 <= len(out.tokens) <= 4
        got += out.tokens
        pending = out.tokens[-1]
    assert got[:20] == want
    # sampled generation on another slot, with top-k / top-p and penalties
    s2 = ses.acquire(p[:30], 32)
    ses.begin_prompt(s2, p[:30])
    while not ses.prefill_some(s2, 4096):
        pass
    sp = SamplingParams(temperature=1.0, top_k=20, top_p=0.95, repetition_penalty=1.1, seed=7)
    t, _ = ses.sample_prompt(s2, sp)
    outs = ses.generate([StepReq(s2, t, 8, 0, sp)], k=2)
    assert all(0 <= x < cfg.vocab for x in outs[0].tokens) and all(lp <= 1e-4 for lp in outs[0].logprobs)
    ids, lps = ses.top_logprobs(0, 5)
    assert len(ids) == 5 and lps[0] >= lps[-1]


def _ready(ses, cfg, slot_prompt):
    for p in slot_prompt:
        s = ses.acquire(p, 64)
        ses.begin_prompt(s, p)
        while not ses.prefill_some(s, 4096):
            pass
        ses.set_stop_tokens(s, [])
        yield s


def test_generate_batches_requests_into_one_step():
    """Three requests through one generate() call per step (one draft chain, one verification step, one sampler call, one
    accept launch) emit token for token what each request emits alone."""
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    cfg, eng, ses = make(None, slots=3)
    prompts = [prompt_of(cfg, 70 + 9 * i, 30 + i) for i in range(3)]
    slots = list(_ready(ses, cfg, prompts))
    firsts = [ses.sample_prompt(s, SamplingParams())[0] for s in slots]
    want = []
    for p, f in zip(prompts, firsts):
        _, e1, s1 = make(None, slots=1)
        e1.prefill(0, p)
        want.append(e1.generate_greedy(0, f, 12, k=0))
    got, pend = [[] for _ in slots], list(firsts)
    launches = []
    while min(len(g) for g in got) < 12:
        outs = ses.generate([StepReq(s, pend[i], 12, 0, SamplingParams()) for i, s in enumerate(slots)], k=3)
        for i, o in enumerate(outs):
            got[i] += o.tokens
            pend[i] = o.tokens[-1]
        assert ses.last_rows.shape[0] == sum(len(o.tokens) for o in outs)
    for g, w in zip(got, want):
        assert g[:12] == w
    eng.dm.check_error()


def test_penalties_with_drafts_equal_plain_decoding():
    """Presence / frequency / repetition penalties see the pending token and the drafts before a row: generate() with
    drafts emits token for token what it emits without, at a fixed seed."""
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, presence_penalty=0.7, frequency_penalty=0.3,
                        repetition_penalty=1.2, seed=11)
    runs = []
    for k in (0, 3):
        cfg, eng, ses = make(None, slots=1)
        p = prompt_of(cfg, 90, 8)
        (s,) = _ready(ses, cfg, [p])
        t, _ = ses.sample_prompt(s, sp)
        out, pending = [], t
        while len(out) < 16:
            o = ses.generate([StepReq(s, pending, 16 - len(out), 0, sp)], k=k, force_accept=None)[0]
            out += o.tokens
            pending = o.tokens[-1]
        runs.append([t] + out[:16])
    assert runs[0] == runs[1]


def test_forced_acceptance_keeps_the_slot_consistent():
    """Accepting drafts by decree (the benchmark mode) leaves a slot whose state is that of its token list: the next
    step's logits equal those of an engine that simply prefilled those tokens."""
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    cfg, eng, ses = make(None, slots=2)
    prompts = [prompt_of(cfg, 75, 41), prompt_of(cfg, 66, 42)]
    slots = list(_ready(ses, cfg, prompts))
    pend = [ses.sample_prompt(s, SamplingParams())[0] for s in slots]
    for step in range(4):
        outs = ses.generate([StepReq(s, pend[i], 32, 0, SamplingParams()) for i, s in enumerate(slots)], k=3, force_accept=2)
        for i, o in enumerate(outs):
            assert len(o.tokens) == 3
            pend[i] = o.tokens[-1]
    for i, s in enumerate(slots):
        _, e1, _ = make(None, slots=1)
        e1.prefill(0, eng.slot[s].tokens)
        e1.decode([0], [pend[i]])
        want = e1.dm.buf["logits"][0].clone()
        eng.decode([s], [pend[i]])
        got = eng.dm.buf["logits"][0]
        assert float((got - want).abs().max() / want.abs().max()) < 3e-2, i


def test_device_snapshots_at_prompt_end_and_message_boundaries():
    """A slot that has generated past its prompt goes back to the device snapshot taken at the prompt's end when the same
    prompt comes again (regenerate) or comes with a different last message: the reused length is the snapshot's position,
    not the last stored block's, and what follows equals a computation from scratch."""
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session.session import StepReq
    cfg, eng, ses = make(None, slots=1)
    ses.snap_min_gap = 256
    boundary = 999
    ses.set_boundary_token(boundary)
    sys_msg = [t if t != boundary else 5 for t in prompt_of(cfg, 330, 51)]
    msg1 = [boundary] + [t if t != boundary else 6 for t in prompt_of(cfg, 90, 52)]
    p1 = sys_msg + msg1
    s = ses.acquire(p1, 32)
    assert ses.begin_prompt(s, p1) == 0
    while not ses.prefill_some(s, 4096):
        pass
    # captures: at the message boundary (position 330, not a block boundary) and at the prompt's end
    assert sorted(v.n for v in ses.vram_snaps) == [330, len(p1)]
    first, _ = ses.sample_prompt(s, SamplingParams())
    pending = first
    for _ in range(3):
        pending = ses.generate([StepReq(s, pending, 8, 0, SamplingParams())], k=2)[0].tokens[-1]
    ses.release(s)
    # the same prompt again: everything is reused, the first token is the same
    assert ses.acquire(p1, 32) == s and ses.begin_prompt(s, p1) == len(p1)
    assert ses.prefill_some(s, 4096)
    again, _ = ses.sample_prompt(s, SamplingParams())
    assert again == first
    ses.release(s)
    # the system prompt with a different message: back to the boundary snapshot (330 > the 256 tokens the store holds)
    msg2 = [boundary] + [t if t != boundary else 7 for t in prompt_of(cfg, 70, 53)]
    p2 = sys_msg + msg2
    assert ses.acquire(p2, 32) == s and ses.begin_prompt(s, p2) == 330
    while not ses.prefill_some(s, 4096):
        pass
    got = ses.slots[s].logits.clone()
    _, e2, s2 = make(None, slots=1)
    e2.prefill(0, p2)
    want = e2.dm.buf["logits"][0]
    assert float((got - want).abs().max() / want.abs().max()) < 3e-2


def test_plain_stretches_and_mtp_catch_up_keep_the_output_exact():
    """Random weights accept no draft, so the acceptance average falls until drafting stops paying: the session then
    decodes a stretch of plain steps, catches the skipped MTP rows up in batched passes, probes with drafts again and,
    failing again, starts a longer stretch.  The tokens equal plain greedy decoding throughout."""
    from qwb200.engine.sampling import SamplingParams
    from qwb200.session import session as SS
    cfg, eng, ses = make(None, slots=1)
    p = prompt_of(cfg, 64, 11)
    s = ses.acquire(p, 400)
    ses.begin_prompt(s, p)
    while not ses.prefill_some(s, 4096):
        pass
    ses.set_stop_tokens(s, [])
    first, _ = ses.sample_prompt(s, SamplingParams())
    cfg2, eng2, ses2 = make(None, slots=1)
    eng2.prefill(0, p)
    n_new = 150
    want = eng2.generate_greedy(0, first, n_new, k=0)
    got, pending, drafted, plain, stretches = [], first, 0, 0, []
    si = ses.slots[s]
    while len(got) < n_new:
        before = si.plain_left
        out = ses.generate([SS.StepReq(s, pending, n_new - len(got), 0, SamplingParams())], k=3)[0]
        if before == 0 and si.plain_left > 0:
            stretches.append(si.plain_left + 1 if si.plain_left < si.plain_stretch - SS.PLAIN_GROW else si.plain_left)
        plain += 1 if (before > 0 or si.plain_left > 0) else 0
        got += out.tokens
        pending = out.tokens[-1]
    eng.dm.check_error()
    assert got[:n_new] == want
    assert len(stretches) >= 2 and plain >= SS.PLAIN_FIRST                # drafting stopped, was probed again, stopped again
    assert si.plain_stretch > SS.PLAIN_FIRST + SS.PLAIN_GROW - 1          # the second stretch is longer than the first
    assert ses.catch_up_rows >= SS.PLAIN_FIRST - 1                         # the first stretch's MTP rows were run when drafting resumed
