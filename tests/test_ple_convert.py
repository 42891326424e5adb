"""PLE table converter: raw bf16 shards -> every sidecar layout -> readable by PleTable with the expected error."""
import numpy as np
import pytest
import torch

from qwb200.models.config import ModelConfig
from qwb200.models.ple import PleTable
from qwb200.tools import ple_convert as pc


def _raw(tmp_path, cfg, shards=2, rows=96):
    g = torch.Generator().manual_seed(1)
    xs = []
    d = tmp_path / "raw"
    d.mkdir()
    for i in range(shards):
        x = (torch.randn(rows, cfg.ngram_dim, generator=g) * 0.3).to(torch.bfloat16)
        x.view(torch.int16).numpy().astype(np.int16).tofile(str(d / f"shard_{i}.bf16"))
        xs.append(x.float())
    return str(d), torch.cat(xs)


@pytest.mark.parametrize("layout,tol", [("bf16", 0.0), ("int8", 0.005), ("int4", 0.08), ("f8", 0.07)])
def test_convert_raw_to_layout(tmp_path, layout, tol):
    cfg = ModelConfig()
    src, x = _raw(tmp_path, cfg)
    dst = str(tmp_path / layout)
    worst = pc.convert(src, dst, layout, cfg.ngram_dim)
    assert worst <= tol
    t = PleTable.load(cfg, dst)
    assert t.rows == x.shape[0] and t.layout == layout and len(t.shards) == 2
    ids = torch.tensor([0, 5, 95, 96, 191])
    got = t.rows_f32(ids)
    assert (got - x[ids]).abs().max() <= tol * x.abs().max() + 1e-7


def test_convert_sidecar_to_sidecar_and_resume(tmp_path, capsys):
    cfg = ModelConfig()
    src, x = _raw(tmp_path, cfg)
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    pc.convert(src, a, "int8", cfg.ngram_dim)
    assert pc.main(["--src", a, "--dst", b, "--layout", "f8", "--width", str(cfg.ngram_dim), "--worker", "0/2"]) == 0
    assert pc.main(["--src", a, "--dst", b, "--layout", "f8", "--width", str(cfg.ngram_dim), "--worker", "1/2"]) == 0
    capsys.readouterr()
    pc.convert(a, b, "f8", cfg.ngram_dim)                  # everything exists: nothing converted
    assert "shard" not in capsys.readouterr().out
    t = PleTable.load(cfg, b)
    assert (t.rows_f32(torch.arange(192)) - x).abs().max() < 0.08 * x.abs().max()
