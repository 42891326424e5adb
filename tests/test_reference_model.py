"""The fp32 oracle: self-consistency (chunked == one pass == token by token), selection rules."""
import numpy as np
import torch

from qwb200.models.config import ModelConfig
from qwb200.models.ple import PleTable
from qwb200.models.reference import RefModel, greedy_generate
from qwb200.models.weights import synth_weights


def make(cfg, seed=0):
    w = synth_weights(cfg, seed=seed)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=seed)
    return RefModel(cfg, w, table)


def test_chunked_equals_single_pass_and_token_by_token():
    cfg = ModelConfig.tiny()
    m = make(cfg)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab, (90,), generator=g).tolist()   # > idx_budget (64): top-k selection is live
    toks[40] = cfg.eos
    st = m.new_state()
    full = m.forward(st, toks, all_logits=True)
    st2 = m.new_state()
    parts = [m.forward(st2, toks[a:b], all_logits=True) for a, b in ((0, 33), (33, 34), (34, 90))]
    chunked = torch.cat(parts)
    assert torch.allclose(full, chunked, atol=2e-4, rtol=1e-3)
    st3 = m.new_state()
    last = None
    for t in toks:
        last = m.forward(st3, [t])
    assert torch.allclose(full[-1], last[0], atol=2e-4, rtol=1e-3)
    assert torch.argmax(full[-1]) == torch.argmax(last[0])
    assert st.n_tokens == 90 and len(st.qsa[0].ck) == 22


def test_selection_is_dense_below_budget_and_topk_above():
    cfg = ModelConfig.tiny()
    m = make(cfg)
    iq = torch.randn(cfg.idx_heads, cfg.idx_dim)
    ck = torch.randn(40, cfg.idx_dim)
    assert m.qsa_select(iq, ck, 50).tolist() == list(range(51))            # nb = 12 <= 16
    sel = m.qsa_select(iq, ck, 101)                                        # nb = 25 > 16
    assert len(sel) == 16 * 4 + 2 and sel[-2:].tolist() == [100, 101]
    sc = torch.relu(ck[:25] @ iq.T).sum(-1)
    best = set(torch.topk(sc, 16).indices.tolist())
    assert {int(s) // 4 for s in sel[:-2]} == best
    # ties go to the lowest index
    ck2 = torch.zeros(40, cfg.idx_dim)
    sel2 = m.qsa_select(iq, ck2, 101)
    assert {int(s) // 4 for s in sel2[:-2]} == set(range(16))


def test_greedy_and_mtp_run():
    cfg = ModelConfig.tiny(n_layers=2, layer_types=("gdn", "qsa"))
    m = make(cfg, seed=1)
    out, logits = greedy_generate(m, [1, 2, 3, 4, 5], 4)
    assert len(out) == 4 and logits.shape == (4, cfg.vocab) and torch.isfinite(logits).all()
    st = m.new_state()
    _, hid = m.forward(st, [1, 2, 3, 4, 5], return_hidden=True)
    dl, h2 = m.mtp_forward(st, hid[:-1], [2, 3, 4, 5], base=0)
    assert dl.shape == (4, cfg.vocab) and h2.shape == (4, cfg.hch) and torch.isfinite(dl).all()


def test_layer_dump_matches_final_state():
    cfg = ModelConfig.tiny(n_layers=2, layer_types=("gdn", "qsa"))
    m = make(cfg)
    m.dump_layers = []
    st = m.new_state()
    _, hid = m.forward(st, [5, 6, 7], return_hidden=True)
    assert len(m.dump_layers) == 2 and torch.equal(m.dump_layers[-1], hid)
