"""Diagnostic tools that need a GPU: divergence of prefill and decode by depth."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_layer_diff_stays_at_rounding_level_at_every_depth():
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    from qwb200.tools.layer_diff import depth_divergence
    cfg = ModelConfig.tiny()
    w = synth_weights(cfg, seed=11)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=11)
    eng = Engine.from_weights(cfg, w, table, EngineOptions(slots=2, slot_tokens=512, use_graphs=False, prefill_chunk=128))
    toks = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    rows = depth_divergence(eng, toks)
    assert [r["depth"] for r in rows] == list(range(1, cfg.n_layers + 1))
    assert {r["layer_kind"] for r in rows} == {"gdn", "qsa"}
    for r in rows:
        assert r["rel"] < 3e-2 and r["kl"] < 1e-2, r
    # the full depth agrees with a plain prefill-vs-decode comparison: the probes left slot 1's state untouched
    full = depth_divergence(eng, toks, depths=[cfg.n_layers])[0]
    assert abs(full["rel"] - rows[-1]["rel"]) < 1e-3
    with pytest.raises(ValueError):
        depth_divergence(eng, toks[:8])
