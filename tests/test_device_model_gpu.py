"""End to end: the native runtime's batched step against the fp32 oracle on tiny models."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def build(cfg, seed=0, slots=2, slot_tokens=512, **kw):
    from qwb200.engine.device_model import DeviceModel
    from qwb200.models.ple import PleTable
    from qwb200.models.reference import RefModel
    from qwb200.models.weights import synth_weights
    w = synth_weights(cfg, seed=seed)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=seed)
    ref = RefModel(cfg, w, table)
    dm = DeviceModel(cfg, slots=slots, slot_tokens=slot_tokens, **kw)
    dm.set_globals(w)
    for L in range(cfg.n_layers):
        dm.set_layer(L, w)
    dm.set_ple_table(table)
    return ref, dm


def ctx3_for(cfg, hist, toks):
    """n-gram context rows for tokens appended after ``hist``."""
    seq = list(hist) + list(toks)
    out = np.full((len(toks), 3), -1, dtype=np.int32)
    for i in range(len(toks)):
        p = len(hist) + i
        out[i, 0] = seq[p]
        if p >= 1:
            out[i, 1] = seq[p - 1]
        if p >= 2:
            out[i, 2] = seq[p - 2]
    return out


def run_seq(dm, cfg, toks, slot=0, start=0, batch=1, hist=(), graph=False):
    """Feed tokens through the device model ``batch`` rows at a time; return logits of every row."""
    outs = []
    hist = list(hist)
    i = 0
    while i < len(toks):
        chunk = toks[i:i + batch]
        pos = list(range(start + i, start + i + len(chunk)))
        dm.step(chunk, [slot] * len(chunk), pos, ctx3_for(cfg, hist, chunk), graph=graph)
        torch.cuda.synchronize()
        outs.append(dm.buf["logits"][:len(chunk)].clone())
        hist += chunk
        i += len(chunk)
    return torch.cat(outs)


def rel(a, b):
    return float((a - b).abs().max() / b.abs().max())


def test_decode_matches_oracle_token_by_token_and_batched():
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.tiny()
    ref, dm = build(cfg)
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab, (100,), generator=g).tolist()     # beyond the budget of 64 tokens
    toks[30] = cfg.eos
    st = ref.new_state()
    want = ref.forward(st, toks, all_logits=True)
    got1 = run_seq(dm, cfg, toks, slot=0, batch=1).cpu()
    assert rel(got1, want) < 3e-2
    agree = (got1.argmax(-1) == want.argmax(-1)).float().mean()
    assert agree > 0.9
    # batched rows (runs of one slot) on another slot: same logits as one row at a time, bit for bit
    got7 = run_seq(dm, cfg, toks, slot=1, batch=7).cpu()
    assert rel(got7, want) < 3e-2
    assert torch.equal(got7, got1)


def test_two_slots_interleaved_rows_are_independent():
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.tiny(n_layers=2, layer_types=("gdn", "qsa"))
    ref, dm = build(cfg, seed=3)
    a = [5, 9, 200, 31, 77, 600]
    b = [8, 8, 8, 901, 2, 44]
    la = run_seq(dm, cfg, a, slot=0).cpu()
    dm.reset_slot(0)
    # same sequences decoded as mixed batches: rows [a_i, b_i]
    ha, hb, outs_a, outs_b = [], [], [], []
    for i in range(len(a)):
        c3 = np.concatenate([ctx3_for(cfg, ha, [a[i]]), ctx3_for(cfg, hb, [b[i]])])
        dm.step([a[i], b[i]], [0, 1], [i, i], c3)
        torch.cuda.synchronize()
        outs_a.append(dm.buf["logits"][0].clone())
        outs_b.append(dm.buf["logits"][1].clone())
        ha.append(a[i]); hb.append(b[i])
    assert torch.equal(torch.stack(outs_a).cpu(), la)
    stb = ref.new_state()
    wb = ref.forward(stb, b, all_logits=True)
    assert rel(torch.stack(outs_b).cpu(), wb) < 3e-2


def test_cuda_graph_replay_equals_direct_launch():
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.tiny(n_layers=2, layer_types=("gdn", "qsa"))
    ref, dm = build(cfg, seed=4)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8]
    direct = run_seq(dm, cfg, toks, slot=0).cpu()
    viag = run_seq(dm, cfg, toks, slot=1, graph=True).cpu()
    assert torch.equal(direct, viag)


def test_full_shape_slice_logits():
    """The two-layer slice at the model's real per-layer shapes (GDN + QSA + MoE + HC + PLE)."""
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.slice2()
    cfg = ModelConfig(**{**cfg.__dict__, "n_experts": 64, "vocab": 4096, "eos": 4000, "image_pad": 4001,
                         "video_pad": 4002, "ngram_vocab_base": 3000})
    ref, dm = build(cfg, seed=5, slots=1, slot_tokens=256)
    toks = torch.randint(0, cfg.vocab, (12,), generator=torch.Generator().manual_seed(1)).tolist()
    st = ref.new_state()
    want = ref.forward(st, toks, all_logits=True)
    got = run_seq(dm, cfg, toks, batch=4).cpu()
    assert rel(got, want) < 3e-2


def test_row_batched_prefill_and_chained_decode_match_stepwise():
    """32-row prefill steps and the device-fed chained decode against one-token steps."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=9)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=9)
    toks = torch.randint(0, cfg.vocab, (75,), generator=torch.Generator().manual_seed(2)).tolist()
    a = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False))
    t, want = None, []
    for x in toks:
        t = a.decode([0], [x])[0]
    last_logits = a.dm.buf["logits"][0].clone()
    for _ in range(10):
        want.append(t)
        t = a.decode([0], [t])[0]
    b = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=True, prefill_chunk=0))
    lg = b.prefill(0, toks)
    torch.cuda.synchronize()
    assert rel(lg.cpu(), last_logits.cpu()) < 2e-2
    first = int(b.dm.buf["amax_idx"][b.last_prefill_row])
    assert first == want[0]
    got = [first] + b.decode_chain(0, first, 9)
    assert got == want
    got2 = b.decode_chain(0, got[-1], 3)          # second call replays the captured graph from the start
    assert got2[0] == t                          # `t` is what the stepwise engine produced after want[-1]


def test_token_major_prefill_matches_stepwise_decode():
    """tcgen05-GEMM prefill (chunked) leaves the same slot state and logits as token-by-token decode."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=11)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=11)
    toks = torch.randint(0, cfg.vocab, (300,), generator=torch.Generator().manual_seed(4)).tolist()
    a = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=0))
    for x in toks:
        ta = a.decode([0], [x])[0]
    la = a.dm.buf["logits"][0].clone()
    b = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=128))
    lb = b.prefill(0, toks).clone()
    torch.cuda.synchronize()
    b.dm.check_error()
    assert rel(lb.cpu(), la.cpu()) < 3e-2
    # continue decoding on both: states agree
    agree = 0
    tb = int(b.dm.buf["amax_idx"][b.last_prefill_row])
    for _ in range(12):
        agree += int(ta == tb)
        ta, tb = a.decode([0], [ta])[0], b.decode([0], [tb])[0]
        if ta != tb:
            break
    assert agree >= 8


def test_speculative_greedy_equals_plain_and_mtp_matches_oracle():
    """MTP drafts + verification give exactly the plain greedy tokens; the MTP head's logits match the oracle."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.reference import RefModel
    from qwb200.models.weights import synth_weights
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=13)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=13)
    prompt = torch.randint(0, cfg.vocab, (70,), generator=torch.Generator().manual_seed(6)).tolist()
    plain = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, save_gdn=True))
    plain.prefill(0, prompt)
    first = int(plain.dm.buf["amax_idx"][plain.last_prefill_row])
    want = plain.generate_greedy(0, first, 24, k=0)
    for chunked in (0, 128):
        spec = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, save_gdn=True,
                                                                prefill_chunk=chunked))
        assert spec.mtp
        spec.prefill(0, prompt)
        assert int(spec.dm.buf["amax_idx"][spec.last_prefill_row]) == first
        got = spec.generate_greedy(0, first, 24, k=3)
        assert got == want, (chunked, got, want)
        assert spec.spec_steps <= 24
    # MTP logits against the fp32 oracle: draft for the position after `first`
    ref = RefModel(cfg, w, table)
    st = ref.new_state()
    _, hid = ref.forward(st, prompt, return_hidden=True)
    dl, _ = ref.mtp_forward(st, hid, prompt[1:] + [first], base=0)
    eng = Engine.from_weights(cfg, w, table, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=0))
    eng.prefill(0, prompt)
    eng.dm.buf["hidden_out"][0] = eng.slot[0].mtp_hidden
    eng.dm.mtp_step([first], [0], [len(prompt) - 1])
    torch.cuda.synchronize()
    got = eng.dm.buf["logits"][0].cpu()
    assert rel(got, dl[-1]) < 4e-2


@pytest.mark.gpu
def test_guard_zones_stay_clean_and_catch_a_stray_write():
    """QW_GUARD: every step buffer is followed by 64 KB of 0xA5; a whole prefill + decode run leaves them intact, and a
    write behind a buffer (made from the host here) is reported with the buffer's name."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.utils import settings
    settings.set_current(settings.Settings.from_env({"QW_GUARD": "1"}))
    try:
        eng = Engine.synthetic(ModelConfig.tiny(), EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=128),
                               device="cuda:0", exact=True, ple_rows=4096)
        assert eng.dm.guard_on and len(eng.dm.guards) > 10
        toks = [(i * 11 + 3) % 900 + 5 for i in range(150)]
        eng.prefill(0, toks)
        t = toks[-1]
        for _ in range(6):
            t = eng.decode([0], [t])[0]
        for rows in ([5, 6, 7], [8] * 9):            # multi-row steps too
            eng.decode([0] * len(rows), rows)
        torch.cuda.synchronize()
        eng.dm.check_guards()
        eng.dm.check_error()
        eng.dm.guards["proj"][100] = 0                # what a kernel writing past `proj` would do
        with pytest.raises(RuntimeError, match="'proj'"):
            eng.dm.check_guards()
    finally:
        settings.set_current(settings.Settings.from_env({}))


@pytest.mark.gpu
def test_moe_balance_counters():
    """QW_MOE_STATS: on one rank every pair is local, so each layer counts rows x top_k per step."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.utils import settings
    settings.set_current(settings.Settings.from_env({"QW_MOE_STATS": "1"}))
    try:
        cfg = ModelConfig.tiny()
        eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=256, use_graphs=False, prefill_chunk=0), device="cuda:0",
                               exact=True, ple_rows=4096)
        eng.dm.moe_balance()
        for t in (5, 6, 7):
            eng.decode([0], [t])
        eng.decode([0, 0], [8, 9])
        torch.cuda.synchronize()
        bal = eng.dm.moe_balance()
        assert len(bal) == cfg.n_layers + 1
        assert all(b == (5 * cfg.top_k, 5.0 * cfg.top_k) for b in bal[:cfg.n_layers])
        assert eng.dm.moe_balance()[0] == (0, 0.0)
    finally:
        settings.set_current(settings.Settings.from_env({}))
        eng.dm.lib.qwrt_set_moe_stats(None)


@pytest.mark.gpu
def test_engine_from_checkpoint_with_weight_cache(tmp_path):
    """A checkpoint directory loads through the converted-weights cache: the second start replays rank0.qww and gives
    bit-identical logits; the checkpoint is not read again (it is deleted in between)."""
    import os
    import shutil
    from test_qw_ref import write_checkpoint
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=5)
    table = PleTable.synthetic(cfg, rows=2048, layout="bf16", seed=5)
    d, cdir = str(tmp_path / "ckpt"), str(tmp_path / "cache")
    write_checkpoint(cfg, {k: v for k, v in w.items()}, table, d)
    opts = EngineOptions(slots=1, slot_tokens=256, use_graphs=False, prefill_chunk=0)
    toks = [(i * 7 + 1) % 900 + 5 for i in range(40)]
    a = Engine.from_checkpoint(cfg, d, table, opts, weight_cache_dir=cdir)
    la = a.prefill(0, toks).clone()
    assert os.path.exists(os.path.join(cdir, "rank0.qww"))
    direct = Engine.from_weights(cfg, {k: v for k, v in w.items() if not k.startswith("mtp.")}, table, opts)
    assert torch.equal(direct.prefill(0, toks), la)
    for f in os.listdir(d):                       # keep names, sizes and times (the key), drop the contents' use: replay must not need them
        pass
    b = Engine.from_checkpoint(cfg, d, table, opts, weight_cache_dir=cdir)
    assert torch.equal(b.prefill(0, toks), la)
    shutil.rmtree(cdir)


@pytest.mark.gpu
def test_calibration_hessians(tmp_path):
    """X^T X of every block's input rows, accumulated over two prompts, symmetric, and equal to what the captured inputs give."""
    from qwb200.engine.calibrate import Calibrator
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.tiny()
    eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=128), device="cuda:0",
                           exact=True, ple_rows=4096)
    cal = Calibrator(eng)
    seen = {}
    orig = cal._hook

    def spy(layer, kind, x):
        seen.setdefault((layer, kind), []).append(x.float().clone())
        orig(layer, kind, x)
    cal._hook = spy
    cal.run(0, [(i * 3 + 1) % 900 + 5 for i in range(200)])
    cal.run(0, [(i * 5 + 2) % 900 + 5 for i in range(150)])
    assert len(cal.H) == 2 * cfg.n_layers and all(n == 350 for n in cal.rows.values())
    for k, h in cal.H.items():
        x = torch.cat(seen[k])
        assert torch.allclose(h, x.t() @ x, rtol=1e-4, atol=1e-3) and torch.allclose(h, h.t())
    cal.dump(str(tmp_path))
    from safetensors.torch import load_file
    d = load_file(str(tmp_path / "hessians.safetensors"))
    assert d["layers.0.attn.hessian"].shape == (cfg.hidden, cfg.hidden) and int(d["layers.3.mlp.rows"]) == 350


@pytest.mark.gpu
def test_warmup_captures_graphs_and_memory_plan():
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    eng = Engine.synthetic(ModelConfig.tiny(), EngineOptions(slots=2, slot_tokens=512, use_graphs=True, save_gdn=True), device="cuda:0",
                           exact=True, ple_rows=4096)
    plan = eng.memory_plan()
    assert plan["weights_gb"] > 0 and plan["state_gb"] > 0 and plan["device_free_gb"] > 2
    n = eng.warmup(max_rows=4)
    assert n >= 8 + 1                       # 4 plain + 4 verification graphs + the chained step (+ MTP passes)
    assert eng.slot[0].n == 0
    before = len(eng.dm.graphs)
    ref = Engine.synthetic(ModelConfig.tiny(), EngineOptions(slots=1, slot_tokens=512, use_graphs=False), device="cuda:0", exact=True,
                           ple_rows=4096)
    toks = [(i * 9 + 2) % 900 + 5 for i in range(30)]
    a = [eng.decode([0], [t])[0] for t in toks]
    b = [ref.decode([0], [t])[0] for t in toks]
    assert a == b and len(eng.dm.graphs) == before          # no capture in front of the "user", same tokens as without graphs
