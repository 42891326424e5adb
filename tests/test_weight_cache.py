"""Converted-weights cache file: record, replay in order, key mismatch, strict consumption (no GPU)."""
import os

import pytest
import torch


def test_record_replay_and_invalidation(tmp_path):
    from qwb200.engine.weight_cache import WeightCache, cache_key
    d = str(tmp_path / "model")
    os.makedirs(d)
    open(os.path.join(d, "a.safetensors"), "wb").write(b"x" * 100)
    k1 = cache_key(d, 0, 2, "H=256")
    assert k1 == cache_key(d, 0, 2, "H=256") and k1 != cache_key(d, 1, 2, "H=256") and k1 != cache_key(d, 0, 2, "H=512")
    layer = {"is_qsa": True, "Wproj": torch.randn(7, 16).to(torch.bfloat16), "attn_hc": {"w1": torch.randn(4, 5), "n_inj": 4},
             "w13": torch.randint(0, 2**31 - 1, (3, 8), dtype=torch.int32), "empty": torch.zeros(0, 4)}
    cdir = str(tmp_path / "cache")
    c = WeightCache(cdir, 0, k1)
    assert not c.replaying
    c.put("globals", {"embed": torch.arange(12, dtype=torch.float32).view(3, 4)})
    c.put("layer0", layer)
    assert not os.path.exists(os.path.join(cdir, "rank0.qww"))          # only published when complete
    c.close()
    r = WeightCache(cdir, 0, k1)
    assert r.replaying
    g = r.get("globals", "cpu")
    l0 = r.get("layer0", "cpu")
    r.close()
    assert torch.equal(g["embed"], torch.arange(12, dtype=torch.float32).view(3, 4))
    assert l0["is_qsa"] is True and l0["attn_hc"]["n_inj"] == 4 and l0["empty"].shape == (0, 4)
    for k in ("Wproj", "w13"):
        assert torch.equal(l0[k], layer[k]) and l0[k].dtype == layer[k].dtype
    assert torch.equal(l0["attn_hc"]["w1"], layer["attn_hc"]["w1"])
    # wrong order / unconsumed records are errors
    r = WeightCache(cdir, 0, k1)
    with pytest.raises(RuntimeError, match="expected record"):
        r.get("layer0", "cpu")
    r = WeightCache(cdir, 0, k1)
    r.get("globals", "cpu")
    with pytest.raises(RuntimeError, match="not consumed"):
        r.close()
    # a touched checkpoint file changes the key: the old file is ignored and recorded anew
    os.utime(os.path.join(d, "a.safetensors"), ns=(1, 1))
    k2 = cache_key(d, 0, 2, "H=256")
    assert k2 != k1 and not WeightCache(cdir, 0, k2).replaying
