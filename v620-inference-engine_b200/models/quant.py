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


def _pack_q4(q: torch.Tensor) -> torch.Tensor:
    """int values in [-8, 7] ``[out, in]`` -> checkpoint-order words ``[out, in/8]``."""
    out, inn = q.shape
    n = (q.to(torch.int64) + 8).reshape(out, inn // 8, 8)
    shifts = torch.arange(8, dtype=torch.int64, device=q.device) * 4
    packed = (n << shifts).sum(dim=-1)
    return torch.where(packed >= 2**31, packed - 2**32, packed).to(torch.int32)


def quantize_q4_gptq(w: torch.Tensor, hessian: torch.Tensor, group: int = QGROUP, *, damp: float = 0.01, block: int = 128,
                     scale_dtype=torch.float16):
    """GPTQ form of :func:`quantize_q4`: the same format (amax/7 group scales, values -8..7), but every column's rounding
    error is pushed onto the columns not yet quantised through the inverse of ``hessian`` = X^T X of the matrix's input
    (as accumulated by ``engine.calibrate.Calibrator``), so that ``||X W^T - X Wq^T||`` shrinks instead of ``||W - Wq||``.
    A group's scale is taken when its first column is reached, from the weights as updated so far.
    (The reference's tools/gptq_int8.py:60-125 does this for its int8 g32 decode copies; here it targets the q4 g128
    expert / MTP format the kernels read.)  Returns (packed, scale) like ``quantize_q4``."""
    out, inn = w.shape
    assert inn % group == 0 and hessian.shape == (inn, inn)
    W = w.double().clone()
    H = hessian.double().clone()
    dead = torch.diagonal(H) <= 0
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    H += torch.eye(inn, dtype=H.dtype, device=H.device) * (damp * torch.diagonal(H).mean())
    L = torch.linalg.cholesky(H)
    U = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)       # upper factor of H^-1: row i drives columns >= i
    Q = torch.zeros(out, inn, dtype=torch.int32, device=w.device)
    scale = torch.zeros(out, inn // group, dtype=scale_dtype, device=w.device)
    sc = inv = None
    for b0 in range(0, inn, block):
        b1 = min(inn, b0 + block)
        Wb = W[:, b0:b1].clone()
        Eb = torch.zeros_like(Wb)
        Ub = U[b0:b1, b0:b1]
        for i in range(b1 - b0):
            col = b0 + i
            if col % group == 0:
                # the columns of this group inside the block carry the updates of everything before them
                g1 = min(col + group, b1)
                cur = torch.cat([Wb[:, i:i + (g1 - col)], W[:, g1:col + group]], dim=1) if g1 < col + group else Wb[:, i:i + group]
                s = (cur.abs().amax(dim=1) / 7.0).to(scale_dtype)
                scale[:, col // group] = s
                sc = s.double()
                inv = torch.where(sc > 0, 1.0 / sc, torch.zeros_like(sc))
            x = Wb[:, i]
            q = torch.round(x * inv).clamp_(-8, 7)
            Q[:, col] = q.to(torch.int32)
            e = (x - q * sc) / Ub[i, i]
            Wb[:, i:] -= e.unsqueeze(1) * Ub[i, i:].unsqueeze(0)
            Eb[:, i] = e
        W[:, b1:] -= Eb @ U[b0:b1, b1:]
    return _pack_q4(Q), scale
