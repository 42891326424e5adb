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


def test_media_tokens_through_prefill_and_prefix_cache():
    """An image's tokens enter the model as the tower's output: same image -> same logits and a cache hit, another
    image -> other logits; the ids come from the content hash, so the prefix cache sees through them."""
    import numpy as np
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.vision import VisionConfig, VisionEncoder, VisionFrontend, synth_vision_weights
    cfg = ModelConfig.tiny()
    eng = Engine.synthetic(cfg, EngineOptions(slots=2, slot_tokens=512, use_graphs=False, prefill_chunk=128), device="cuda:0",
                           exact=True, ple_rows=4096)
    vc = VisionConfig(depth=1, out_dim=cfg.hidden)
    fe = VisionFrontend(VisionEncoder(vc, synth_vision_weights(vc, seed=2), "cuda:0"))
    eng.vision_lookup = fe.lookup
    h, w = 4, 6
    n_img = h * w // 4
    rng = np.random.default_rng(0)
    img_a = rng.standard_normal((h * w, vc.patch_in)).astype(np.float32).clip(-1, 1)
    img_b = rng.standard_normal((h * w, vc.patch_in)).astype(np.float32).clip(-1, 1)
    text = [5 + (i * 7) % 900 for i in range(40)]

    def prompt(img, hsh):
        toks = text[:20] + [cfg.image_pad] * n_img + text[20:]
        fe.add_media(toks, hsh, False, 1, h, w, img, [20])
        return toks
    pa, pa2, pb = prompt(img_a, 111), prompt(img_a, 111), prompt(img_b, 222)
    assert pa == pa2 and pa != pb and all(t < 0 and (-t) & 1 for t in pa[20:20 + n_img])
    la = eng.prefill(0, pa).clone()
    eng.reset(0)
    la2 = eng.prefill(0, pa2).clone()
    lb = eng.prefill(1, pb).clone()
    torch.cuda.synchronize()
    eng.dm.check_error()
    assert torch.isfinite(la).all() and torch.equal(la, la2)
    assert fe.cache.hits >= 1 and fe.cache.misses == 2
    assert rel(lb, la) > 1e-3
    # a text-only prompt of the same shape (pad tokens, no image) differs too: the embeddings really come from the tower
    eng.reset(0)
    lt = eng.prefill(0, text[:20] + [cfg.image_pad] * n_img + text[20:]).clone()
    assert rel(lt, la) > 1e-3
    with pytest.raises(ValueError):
        eng.vision_lookup = None
        eng.reset(0)
        eng.prefill(0, pa)
