"""Tensor-level Python wrappers of the native kernel launchers.

Thin: they check shapes/dtypes, pass raw pointers and the current CUDA stream, and never fall
back to PyTorch — a missing native library on a GPU machine raises.  The engine itself calls the
native runtime (one call per step); these wrappers serve tests, tools and the prefill scheduler.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import lib as qlib


def _s() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def gemv_bf16(W: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
              nsplit: int = 1, splits: Tuple[int, int, int] = (0, 0, 0), N: Optional[int] = None,
              K: Optional[int] = None, ldw: Optional[int] = None, ldy: Optional[int] = None) -> torch.Tensor:
    """y[m][n] = sum_k W[n][k] x[m][k]; W bf16 [N, K], x bf16 [M, K], y fp32 [M, N]."""
    lib = qlib.load(required=True)
    assert W.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and W.is_cuda and x.is_cuda
    M = x.shape[0]
    N = W.shape[0] if N is None else N
    K = W.shape[1] if K is None else K
    ldw = W.stride(0) if ldw is None else ldw
    if out is None:
        out = torch.empty((M, N if ldy is None else ldy), dtype=torch.float32, device=x.device)
    ldy = out.stride(0) if ldy is None else ldy
    qlib.check(lib.qwk_gemv_bf16(_p(W), _p(x), _p(out), None, N, K, M, ldw, x.stride(0), ldy, int(accumulate), nsplit,
                                 splits[0], splits[1], splits[2], _s()), "gemv_bf16")
    return out


def row_reduce(logits: torch.Tensor, idx0: int = 0, lse: bool = True):
    lib = qlib.load(required=True)
    M, V = logits.shape
    dev = logits.device
    val = torch.empty(M, dtype=torch.float32, device=dev)
    idx = torch.empty(M, dtype=torch.int32, device=dev)
    mx = torch.empty(M, dtype=torch.float32, device=dev) if lse else None
    sm = torch.empty(M, dtype=torch.float32, device=dev) if lse else None
    qlib.check(lib.qwk_row_reduce(_p(logits), logits.stride(0), V, idx0, M, _p(val), _p(idx), _p(mx), _p(sm), _s()),
               "row_reduce")
    return val, idx, mx, sm


def qsa_select(scores: torch.Tensor, pos: torch.Tensor, ratio: int, topk: int):
    """scores fp32 [M, cap], pos int32 [M] -> (sel int32 [M, topk] ascending, sel_n int32 [M]; -1 = dense)."""
    lib = qlib.load(required=True)
    M = scores.shape[0]
    sel = torch.full((M, topk), -1, dtype=torch.int32, device=scores.device)
    sel_n = torch.zeros(M, dtype=torch.int32, device=scores.device)
    qlib.check(lib.qwk_qsa_select(_p(scores), scores.stride(0), M, _p(pos), ratio, topk, _p(sel), _p(sel_n), _s()),
               "qsa_select")
    return sel, sel_n


def moe_route(rs: torch.Tensor, E: int, top_k: int, SF: int, e_first: int = 0, e_local: Optional[int] = None):
    lib = qlib.load(required=True)
    M = rs.shape[0]
    dev = rs.device
    pe = torch.empty((M, top_k), dtype=torch.int32, device=dev)
    pw = torch.empty((M, top_k), dtype=torch.float32, device=dev)
    sh = torch.empty((M, SF), dtype=torch.bfloat16, device=dev)
    qlib.check(lib.qwk_moe_route(_p(rs), rs.stride(0), M, E, top_k, SF, e_first, E if e_local is None else e_local,
                                 _p(pe), _p(pw), _p(sh), _s()), "moe_route")
    return pe, pw, sh


def moe_experts_pair(w13, s13, w2, s2, x, pair_expert, pair_w, F: int, H: int, shared_down=None, sh_h=None):
    """Routed experts for rows x bf16 [M, H] (+ optional shared expert): returns fp32 [M, H]."""
    lib = qlib.load(required=True)
    M, top_k = pair_expert.shape
    dev = x.device
    h = torch.empty((M * top_k, F), dtype=torch.bfloat16, device=dev)
    out = torch.empty((M, H), dtype=torch.float32, device=dev)
    qlib.check(lib.qwk_moe_gate_up_pair(_p(w13), _p(s13), _p(x), x.stride(0), _p(pair_expert), M, top_k, F, H, _p(h), _s()),
               "moe_gate_up_pair")
    SF = 0 if sh_h is None else sh_h.shape[1]
    qlib.check(lib.qwk_moe_down_combine(_p(w2), _p(s2), _p(h), _p(pair_expert), _p(pair_w), M, top_k, F, H,
                                        _p(shared_down), 0 if shared_down is None else shared_down.stride(0),
                                        _p(sh_h), SF, _p(out), H, _s()), "moe_down_combine")
    return out


def gemm_bf16_tc(A: torch.Tensor, W: torch.Tensor, out_dtype=torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ W.T on the tcgen05 tensor cores.  A bf16 [T, K], W bf16 [N, K]; C fp32 or bf16 [T, N]."""
    lib = qlib.load(required=True)
    assert A.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and A.is_cuda and W.is_cuda
    assert A.stride(1) == 1 and W.stride(1) == 1
    T, Kd = A.shape
    N = W.shape[0]
    if out is None:
        out = torch.empty((T, N), dtype=out_dtype, device=A.device)
    assert out.dtype in (torch.float32, torch.bfloat16) and out.stride(1) == 1
    qlib.check(lib.qwk_gemm_bf16_tc(_p(A), _p(W), _p(out), T, N, Kd, A.stride(0), W.stride(0), out.stride(0),
                                    1 if out.dtype == torch.bfloat16 else 0, _s()), "gemm_bf16_tc")
    return out
