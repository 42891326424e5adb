"""Qwen3-VL vision tower on the device: depth 27, width 1152, 16 heads x 72, MLP 4304, patches of 3x2x16x16 = 1536
values, a learned 48x48 position table interpolated bilinearly to the image's patch grid, 2-D rotary attention,
and a 2x2 merger to the language model's width (reference: src/vision/vision_weights.hpp:13-17,
src/vision/vision_encoder.hip:71-145).

One slice (an image, or one temporal patch of a video) is encoded per call: attention is over the slice's
patches only.  All seven products per block (patch embed, qkv, proj, fc1, fc2, merger fc1/fc2) run on the
tcgen05 GEMM (``ops/csrc/gemm_tc.cu``); everything between them is in ``ops/csrc/vision.cu``.  The residual stream
is fp32, GEMM operands bf16.  Weights come from ``model.visual.*`` of the checkpoint
(src/vision/vision_weights.cpp:33-63)."""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np
import torch

PREFIX = "model.visual."


@dataclass(frozen=True)
class VisionConfig:
    depth: int = 27
    dim: int = 1152
    heads: int = 16
    mlp: int = 4304
    out_dim: int = 2560
    patch_in: int = 3 * 2 * 16 * 16
    merge: int = 2
    grid_side: int = 48
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads


def synth_vision_weights(cfg: VisionConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Random weights with the checkpoint's names and shapes (bf16, as stored)."""
    g = torch.Generator().manual_seed(seed)
    D, M, DM = cfg.dim, cfg.mlp, cfg.dim * cfg.merge ** 2

    def mat(n, k, scale=None):
        return (torch.randn(n, k, generator=g) * (scale or 1.0 / math.sqrt(k))).to(torch.bfloat16).to(device)

    def vec(n, base=0.0, s=0.05):
        return (base + torch.randn(n, generator=g) * s).to(torch.bfloat16).to(device)
    w = {"patch_embed.proj.weight": mat(D, cfg.patch_in).view(D, 3, 2, 16, 16), "patch_embed.proj.bias": vec(D),
         "pos_embed.weight": mat(cfg.grid_side ** 2, D, 0.1)}
    for b in range(cfg.depth):
        q = f"blocks.{b}."
        w.update({q + "norm1.weight": vec(D, 1.0), q + "norm1.bias": vec(D), q + "norm2.weight": vec(D, 1.0), q + "norm2.bias": vec(D),
                  q + "attn.qkv.weight": mat(3 * D, D), q + "attn.qkv.bias": vec(3 * D), q + "attn.proj.weight": mat(D, D),
                  q + "attn.proj.bias": vec(D), q + "mlp.linear_fc1.weight": mat(M, D), q + "mlp.linear_fc1.bias": vec(M),
                  q + "mlp.linear_fc2.weight": mat(D, M), q + "mlp.linear_fc2.bias": vec(D)})
    w.update({"merger.norm.weight": vec(D, 1.0), "merger.norm.bias": vec(D), "merger.linear_fc1.weight": mat(DM, DM),
              "merger.linear_fc1.bias": vec(DM), "merger.linear_fc2.weight": mat(cfg.out_dim, DM), "merger.linear_fc2.bias": vec(cfg.out_dim)})
    return {PREFIX + k: v for k, v in w.items()}


def slice_positions(h: int, w: int, merge: int, side: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """For the h x w patches of a slice in merge-window order: (row, col) of each patch, and the four taps and
    weights of the bilinear (align-corners) interpolation of the side x side position table at it."""
    i = np.arange(h * w)
    bw = w // merge
    in_col, in_row = i % merge, (i // merge) % merge
    bcol, brow = (i // (merge * merge)) % bw, i // (merge * merge * bw)
    row, col = brow * merge + in_row, bcol * merge + in_col

    def taps(idx, n):
        src = idx.astype(np.float32) * np.float32(side - 1) / np.float32(max(n - 1, 1))
        fl = np.floor(src)
        t0 = np.minimum(fl.astype(np.int64), side - 1)
        t1 = np.minimum(fl.astype(np.int64) + 1, side - 1)
        w1 = (src - fl).astype(np.float32)
        return t0, t1, 1.0 - w1, w1
    y0, y1, wy0, wy1 = taps(row, h)
    x0, x1, wx0, wx1 = taps(col, w)
    idx = np.stack([y0 * side + x0, y0 * side + x1, y1 * side + x0, y1 * side + x1], 1).astype(np.int32)
    wts = np.stack([wy0 * wx0, wy0 * wx1, wy1 * wx0, wy1 * wx1], 1).astype(np.float32)
    pos = np.stack([row, col], 1).astype(np.int32)
    return pos, idx, wts


def vision_reference(cfg: VisionConfig, w: Dict[str, torch.Tensor], patches: torch.Tensor, h: int, wd: int) -> torch.Tensor:
    """Plain fp32 PyTorch forward of one slice (the oracle of the kernels): patches [h*w, 1536] -> [h*w/4, out_dim]."""
    f = lambda n: w[PREFIX + n].float().cpu()
    D, H, hd = cfg.dim, cfg.heads, cfg.head_dim
    L = h * wd
    pos, idx, wts = slice_positions(h, wd, cfg.merge, cfg.grid_side)
    x = patches.float().cpu() @ f("patch_embed.proj.weight").reshape(D, -1).t() + f("patch_embed.proj.bias")
    table = f("pos_embed.weight")
    x = x + (table[torch.from_numpy(idx).long()] * torch.from_numpy(wts)[..., None]).sum(1)
    half, nf = hd // 2, hd // 4
    inv = 10000.0 ** (-2.0 * torch.arange(nf).float() / half)
    ang = torch.cat([torch.from_numpy(pos[:, :1]).float() * inv, torch.from_numpy(pos[:, 1:]).float() * inv], 1)     # [L, half]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rope(t):            # [L, H, hd]
        a, b = t[..., :half], t[..., half:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)
    ln = torch.nn.functional.layer_norm
    for bi in range(cfg.depth):
        q = f"blocks.{bi}."
        xn = ln(x, (D,), f(q + "norm1.weight"), f(q + "norm1.bias"), cfg.eps)
        qkv = xn @ f(q + "attn.qkv.weight").t() + f(q + "attn.qkv.bias")
        qq, kk, vv = [t.view(L, H, hd) for t in qkv.split(D, 1)]
        qq, kk = rope(qq), rope(kk)
        att = torch.softmax(torch.einsum("qhd,khd->hqk", qq, kk) / math.sqrt(hd), -1)
        o = torch.einsum("hqk,khd->qhd", att, vv).reshape(L, D)
        x = x + o @ f(q + "attn.proj.weight").t() + f(q + "attn.proj.bias")
        xn = ln(x, (D,), f(q + "norm2.weight"), f(q + "norm2.bias"), cfg.eps)
        m = torch.nn.functional.gelu(xn @ f(q + "mlp.linear_fc1.weight").t() + f(q + "mlp.linear_fc1.bias"), approximate="tanh")
        x = x + m @ f(q + "mlp.linear_fc2.weight").t() + f(q + "mlp.linear_fc2.bias")
    xn = ln(x, (D,), f("merger.norm.weight"), f("merger.norm.bias"), cfg.eps).view(L // cfg.merge ** 2, D * cfg.merge ** 2)
    m = torch.nn.functional.gelu(xn @ f("merger.linear_fc1.weight").t() + f("merger.linear_fc1.bias"))
    return m @ f("merger.linear_fc2.weight").t() + f("merger.linear_fc2.bias")


def _p(t):
    return C.c_void_p(t.data_ptr())


class VisionEncoder:
    """Device copy of the tower (bf16 matrices, fp32 vectors) + scratch that grows with the largest slice seen."""

    def __init__(self, cfg: VisionConfig, weights: Dict[str, torch.Tensor], device="cuda:0"):
        from ..ops import lib as qlib
        self.cfg, self.dev = cfg, torch.device(device)
        self.lib = qlib.load(required=True)
        self.check = qlib.check
        D = cfg.dim
        mat = lambda n: weights[PREFIX + n].to(self.dev, torch.bfloat16).contiguous()
        vec = lambda n: weights[PREFIX + n].to(self.dev, torch.float32).contiguous()
        self.patch_w = mat("patch_embed.proj.weight").view(D, cfg.patch_in)
        self.patch_b, self.table = vec("patch_embed.proj.bias"), vec("pos_embed.weight")
        self.blocks = []
        for b in range(cfg.depth):
            q = f"blocks.{b}."
            self.blocks.append({k: (mat if k in ("attn.qkv.weight", "attn.proj.weight", "mlp.linear_fc1.weight", "mlp.linear_fc2.weight") else vec)(q + k)
                                for k in ("norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight", "attn.qkv.bias",
                                          "attn.proj.weight", "attn.proj.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias",
                                          "mlp.linear_fc2.weight", "mlp.linear_fc2.bias")})
        self.m_nw, self.m_nb = vec("merger.norm.weight"), vec("merger.norm.bias")
        self.m_fc1, self.m_fc1_b = mat("merger.linear_fc1.weight"), vec("merger.linear_fc1.bias")
        self.m_fc2, self.m_fc2_b = mat("merger.linear_fc2.weight"), vec("merger.linear_fc2.bias")
        self.cap = 0
        self.bytes = sum(t.numel() * t.element_size() for b in self.blocks for t in b.values())

    @classmethod
    def from_checkpoint(cls, model_dir: str, device="cuda:0"):
        """None when the checkpoint has no vision tower."""
        import glob
        import os
        from safetensors import safe_open
        w = {}
        for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
            with safe_open(path, "pt") as f:
                for k in f.keys():
                    if k.startswith(PREFIX):
                        w[k] = f.get_tensor(k)
        if PREFIX + "patch_embed.proj.weight" not in w:
            return None
        depth = 1 + max(int(k.split(".")[3]) for k in w if k.startswith(PREFIX + "blocks."))
        return cls(VisionConfig(depth=depth), w, device)

    def _reserve(self, L: int):
        if L <= self.cap:
            return
        c, dev = self.cfg, self.dev
        self.cap = L
        self.x = torch.empty(L, c.dim, device=dev)
        self.y = torch.empty(L, c.dim, device=dev)
        self.xn = torch.empty(L, c.dim, dtype=torch.bfloat16, device=dev)
        self.qkv = torch.empty(L, 3 * c.dim, dtype=torch.bfloat16, device=dev)
        self.att = torch.empty(L, c.dim, dtype=torch.bfloat16, device=dev)
        self.mlp = torch.empty(L, max(c.mlp, c.patch_in), dtype=torch.bfloat16, device=dev)

    def _gemm(self, A, W, out):
        from ..ops.kernels import gemm_bf16_tc
        return gemm_bf16_tc(A, W, out=out)

    @torch.no_grad()
    def encode(self, patches, h: int, w: int) -> torch.Tensor:
        """patches fp32 [h*w, 1536] (host or device, merge-window order) -> fp32 [h*w/4, out_dim] on the device."""
        c, L, lib = self.cfg, h * w, self.lib
        assert L > 0 and h % c.merge == 0 and w % c.merge == 0, "the patch grid must be a multiple of the merge size"
        self._reserve(L)
        s = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        pos, idx, wts = slice_positions(h, w, c.merge, c.grid_side)
        pos_d, idx_d, wts_d = (torch.from_numpy(a).to(self.dev) for a in (pos, idx, wts))
        pin = torch.as_tensor(patches).to(self.dev, torch.bfloat16).contiguous()
        x, y, xn, qkv, att = self.x[:L], self.y[:L], self.xn[:L], self.qkv[:L], self.att[:L]
        D = c.dim
        self._gemm(pin, self.patch_w, y)
        self.check(lib.qwk_vit_embed(_p(x), _p(y), _p(self.patch_b), _p(self.table), _p(idx_d), _p(wts_d), L, D, s), "vit_embed")
        for b in self.blocks:
            self.check(lib.qwk_vit_layernorm(_p(x), _p(b["norm1.weight"]), _p(b["norm1.bias"]), L, D, C.c_float(c.eps), _p(xn), s), "vit_ln")
            self._gemm(xn, b["attn.qkv.weight"], qkv)
            self.check(lib.qwk_vit_bias_rope(_p(qkv), _p(b["attn.qkv.bias"]), _p(pos_d), L, c.heads, s), "vit_rope")
            self.check(lib.qwk_vit_attention(_p(qkv), L, c.heads, _p(att), s), "vit_attention")
            self._gemm(att, b["attn.proj.weight"], y)
            self.check(lib.qwk_vit_residual_add(_p(x), _p(y), _p(b["attn.proj.bias"]), L, D, 0, s), "vit_add")
            self.check(lib.qwk_vit_layernorm(_p(x), _p(b["norm2.weight"]), _p(b["norm2.bias"]), L, D, C.c_float(c.eps), _p(xn), s), "vit_ln")
            m = self.mlp[:L, :c.mlp]
            self._gemm(xn, b["mlp.linear_fc1.weight"], m)
            if m.is_contiguous():
                self.check(lib.qwk_vit_bias_gelu(_p(m), _p(b["mlp.linear_fc1.bias"]), L, c.mlp, 1, s), "vit_gelu")
            else:           # the scratch rows are wider than the MLP: row by row layout, so run on a compact copy
                mc = m.contiguous()
                self.check(lib.qwk_vit_bias_gelu(_p(mc), _p(b["mlp.linear_fc1.bias"]), L, c.mlp, 1, s), "vit_gelu")
                m = mc
            self._gemm(m, b["mlp.linear_fc2.weight"], y)
            self.check(lib.qwk_vit_residual_add(_p(x), _p(y), _p(b["mlp.linear_fc2.bias"]), L, D, 0, s), "vit_add")
        T, DM = L // c.merge ** 2, D * c.merge ** 2
        self.check(lib.qwk_vit_layernorm(_p(x), _p(self.m_nw), _p(self.m_nb), L, D, C.c_float(c.eps), _p(xn), s), "vit_ln")
        h1 = torch.empty(T, DM, dtype=torch.bfloat16, device=self.dev)
        self._gemm(xn.view(T, DM), self.m_fc1, h1)
        self.check(lib.qwk_vit_bias_gelu(_p(h1), _p(self.m_fc1_b), T, DM, 0, s), "vit_gelu")
        o = torch.empty(T, c.out_dim, device=self.dev)
        self._gemm(h1, self.m_fc2, o)
        out = torch.empty_like(o)
        self.check(lib.qwk_vit_residual_add(_p(out), _p(o), _p(self.m_fc2_b), T, c.out_dim, 1, s), "vit_bias_out")
        return out
