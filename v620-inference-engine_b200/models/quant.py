"""q4 (symmetric int4, group 128) weight format.

Checkpoint layout (compressed-tensors ``pack-quantized``; reference docs/MODEL.md:34-38):
``weight_packed`` int32 ``[out, in/8]`` — word ``c`` holds input columns ``8c..8c+7``, element
``8c+i`` in bits ``4i..4i+3`` stored as ``q+8``; ``weight_scale`` ``[out, in/128]``.

Engine layout: the same words with the nibbles re-ordered so that elements ``2j`` and ``2j+1``
sit at bits ``4j`` and ``16+4j`` (even elements in the low half-word, odd in the high one;
reference src/engine/weight_convert.cpp:61-71).  With that order ``(w >> 4j) & 0x000F000F``
is a pair of consecutive elements, one per 16-bit half, which turns into a packed bf16 pair
``128+n`` by OR-ing ``0x43004300`` — the in-register dequant used by the GEMV and by the
tcgen05 grouped GEMM.
"""
from __future__ import annotations

import torch

QGROUP = 128


def quantize_q4(w: torch.Tensor, group: int = QGROUP, scale_dtype=torch.float16):
    """Quantise ``w [out, in]`` to int4 g``group``: scale = amax/7 rounded to ``scale_dtype``,
    q = clamp(rint(w/scale), -8, 7) (reference weight_convert.cpp:73-90 uses fp16 scales and
    round-half-even ``lrint``).  Returns (packed int32 [out, in/8] in checkpoint order,
    scale [out, in/group])."""
    out, inn = w.shape
    assert inn % group == 0 and group % 8 == 0
    wf = w.float().reshape(out, inn // group, group)
    amax = wf.abs().amax(dim=-1)
    scale = (amax / 7.0).to(scale_dtype)
    sc = scale.float()
    inv = torch.where(sc > 0, 1.0 / sc, torch.zeros_like(sc))
    q = torch.round(wf * inv.unsqueeze(-1)).clamp_(-8, 7).to(torch.int32) + 8   # round-half-even
    q = q.reshape(out, inn // 8, 8)
    shifts = torch.arange(8, dtype=torch.int32, device=w.device) * 4
    packed = (q << shifts).sum(dim=-1, dtype=torch.int64)
    packed = torch.where(packed >= 2**31, packed - 2**32, packed).to(torch.int32)
    return packed, scale


def unpack_q4(packed: torch.Tensor) -> torch.Tensor:
    """Checkpoint-order words -> int8 values in [-8, 7], shape [out, in]."""
    out, words = packed.shape
    shifts = torch.arange(8, dtype=torch.int32, device=packed.device) * 4
    nib = (packed.unsqueeze(-1) >> shifts) & 0xF
    return (nib - 8).to(torch.int8).reshape(out, words * 8)


def dequantize_q4(packed: torch.Tensor, scale: torch.Tensor, group: int = QGROUP) -> torch.Tensor:
    """fp32 weights ``(nibble-8)*scale``."""
    q = unpack_q4(packed).float()
    out, inn = q.shape
    return (q.reshape(out, inn // group, group) * scale.float().unsqueeze(-1)).reshape(out, inn)


def to_engine_order(packed: torch.Tensor) -> torch.Tensor:
    """Re-order nibbles of checkpoint words into the engine order (see module docstring)."""
    w = packed.to(torch.int64) & 0xFFFFFFFF
    r = torch.zeros_like(w)
    for k in range(8):
        nib = (w >> (4 * k)) & 0xF
        bit = 16 + 4 * (k >> 1) if (k & 1) else 4 * (k >> 1)
        r |= nib << bit
    r = torch.where(r >= 2**31, r - 2**32, r)
    return r.to(torch.int32)


def from_engine_order(words: torch.Tensor) -> torch.Tensor:
    w = words.to(torch.int64) & 0xFFFFFFFF
    r = torch.zeros_like(w)
    for k in range(8):
        bit = 16 + 4 * (k >> 1) if (k & 1) else 4 * (k >> 1)
        nib = (w >> bit) & 0xF
        r |= nib << (4 * k)
    r = torch.where(r >= 2**31, r - 2**32, r)
    return r.to(torch.int32)


def random_q4(out: int, inn: int, *, std: float = 0.02, generator=None, device="cpu", scale_dtype=torch.bfloat16):
    """Cheap random q4 weights for full-size synthetic models: nibbles uniform in [1, 15]
    (values -7..7) and a constant-magnitude scale chosen so the dequantised weights have
    standard deviation ``std``.  Returns (packed checkpoint-order int32, scale)."""
    q = torch.randint(-2**31, 2**31 - 1, (out, inn // 8), dtype=torch.int64, generator=generator, device=device)
    packed = q.to(torch.int32)
    # uniform nibble 0..15 -> value -8..7 has std sqrt((16^2-1)/12) = 4.61
    scale = torch.full((out, inn // QGROUP), std / 4.61, dtype=scale_dtype, device=device)
    return packed, scale
