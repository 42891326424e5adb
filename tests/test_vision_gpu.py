"""Vision tower kernels and encoder against the plain fp32 PyTorch forward (the reference checks its tower against
HF fp32 dumps with rel L2 < 2e-2: tests/gpu/test_vision_encoder.hip)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm())


def test_attention_kernel_matches_fp32():
    import ctypes as C
    from qwb200.ops import lib as qlib
    L_ = qlib.load(True)
    heads, hd = 16, 72
    D = heads * hd
    for L in (64, 100, 333):
        g = torch.Generator().manual_seed(L)
        qkv = (torch.randn(L, 3 * D, generator=g) * 0.7).to(torch.bfloat16).cuda()
        out = torch.zeros(L, D, dtype=torch.bfloat16, device="cuda")
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert L_.qwk_vit_attention(C.c_void_p(qkv.data_ptr()), L, heads, C.c_void_p(out.data_ptr()), s) == 0
        q, k, v = [t.float().view(L, heads, hd) for t in qkv.split(D, 1)]
        att = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd), -1)
        ref = torch.einsum("hqk,khd->qhd", att, v).reshape(L, D)
        assert rel(out, ref) < 1.5e-2, (L, rel(out, ref))


def test_encoder_matches_reference_forward():
    from qwb200.vision import VisionConfig, VisionEncoder, synth_vision_weights, vision_reference
    cfg = VisionConfig(depth=3)
    w = synth_vision_weights(cfg, seed=3)
    enc = VisionEncoder(cfg, w, "cuda:0")
    for h, wd in ((8, 12), (6, 4)):
        g = torch.Generator().manual_seed(h * 100 + wd)
        patches = torch.randn(h * wd, cfg.patch_in, generator=g).clamp(-1, 1)
        out = enc.encode(patches, h, wd)
        ref = vision_reference(cfg, w, patches.to(torch.bfloat16), h, wd)
        assert out.shape == (h * wd // 4, cfg.out_dim)
        assert rel(out, ref) < 2e-2, rel(out, ref)
