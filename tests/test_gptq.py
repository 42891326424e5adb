"""GPTQ q4 quantiser: same format as round-to-nearest, lower output error on correlated inputs."""
import torch

from qwb200.models import quant


def test_gptq_beats_round_to_nearest_on_correlated_inputs():
    g = torch.Generator().manual_seed(3)
    K, N, T = 256, 48, 2048
    mix = torch.randn(K, K, generator=g) * 0.2 + torch.eye(K)
    X = torch.randn(T, K, generator=g) @ mix                      # correlated features
    W = torch.randn(N, K, generator=g) * 0.05
    H = X.t() @ X
    p0, s0 = quant.quantize_q4(W)
    p1, s1 = quant.quantize_q4_gptq(W, H)
    assert p1.shape == p0.shape and s1.shape == s0.shape and p1.dtype == torch.int32
    v = quant.unpack_q4(p1)
    assert int(v.min()) >= -8 and int(v.max()) <= 7
    ref = X @ W.t()
    e0 = (X @ quant.dequantize_q4(p0, s0).t() - ref).pow(2).mean()
    e1 = (X @ quant.dequantize_q4(p1, s1).t() - ref).pow(2).mean()
    assert e1 < 0.8 * e0, (float(e0), float(e1))


def test_gptq_identity_hessian_is_round_to_nearest():
    g = torch.Generator().manual_seed(4)
    W = torch.randn(8, 256, generator=g)
    p0, s0 = quant.quantize_q4(W)
    p1, s1 = quant.quantize_q4_gptq(W, torch.eye(256))
    assert torch.equal(s0, s1)
    assert (quant.unpack_q4(p0) != quant.unpack_q4(p1)).float().mean() < 0.01       # ties only


def test_gptq_dead_columns():
    g = torch.Generator().manual_seed(5)
    X = torch.randn(512, 128, generator=g)
    X[:, 7] = 0
    W = torch.randn(4, 128, generator=g)
    p, s = quant.quantize_q4_gptq(W, X.t() @ X)
    assert int(quant.unpack_q4(p)[:, 7].abs().max()) == 0
    assert torch.isfinite(s.float()).all()


def test_gptq_tool_round_trip(tmp_path):
    from safetensors.torch import load_file, save_file
    from qwb200.tools import gptq_q4
    g = torch.Generator().manual_seed(6)
    X = torch.randn(1024, 128, generator=g) @ (torch.randn(128, 128, generator=g) * 0.3 + torch.eye(128))
    W = (torch.randn(16, 128, generator=g) * 0.05).to(torch.bfloat16)
    save_file({"layers.2.mlp.experts.0.up_proj.weight": W, "layers.2.other": W.clone()}, str(tmp_path / "w.safetensors"))
    save_file({"layers.2.moe.hessian": X.t() @ X}, str(tmp_path / "h.safetensors"))
    rc = gptq_q4.main(["--weights", str(tmp_path / "w.safetensors"), "--hessians", str(tmp_path / "h.safetensors"),
                       "--pattern", r"layers\.(\d+)\.mlp\.experts\.\d+\.up_proj\.weight", "--out", str(tmp_path / "o"), "--device", "cpu"])
    assert rc == 0
    o = load_file(str(tmp_path / "o" / "w.safetensors"))
    assert set(o) == {"layers.2.mlp.experts.0.up_proj.weight_packed", "layers.2.mlp.experts.0.up_proj.weight_scale"}
    wq = quant.dequantize_q4(o["layers.2.mlp.experts.0.up_proj.weight_packed"], o["layers.2.mlp.experts.0.up_proj.weight_scale"])
    assert (wq - W.float()).abs().max() < 0.05
