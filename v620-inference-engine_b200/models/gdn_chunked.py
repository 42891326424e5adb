"""Chunked (WY) form of the gated delta rule, in plain PyTorch fp32.

The recurrent form (docs/MODEL.md:108-133 of the reference; its kernel gdn_scan_T walks tokens one by
one, src/kernels/gdn.hip:229-309) is, per value head with state S [dk][dv]:

    S <- a_t S;  u_t = b_t (v_t - S^T k_t);  S <- S + k_t u_t^T;  o_t = S^T q_t

Over a chunk of C tokens with entry state S0 and g_t = sum_{s<=t} log a_s the same numbers come out of
a few dense products (this is what ``ops/csrc/gdn_chunk.cu`` runs on the tensor cores):

    A[t,s] = b_t exp(g_t - g_s) (k_t . k_s)         for s < t, else 0
    (I + A) Wv = diag(b) V        (I + A) Wk = diag(b exp(g)) K      (forward substitution)
    U  = Wv - Wk S0
    P[t,s] = exp(g_t - g_s) (q_t . k_s)             for s <= t, else 0
    O  = diag(exp(g)) Q S0 + P U
    S1 = exp(g_C) S0 + (diag(exp(g_C - g)) K)^T U

``scan_sequential`` and ``scan_chunked`` are the two forms; the CPU tests hold them against each other and
the GPU test holds the kernel against both.
"""
from __future__ import annotations

import torch


def scan_sequential(q, k, v, decay, beta, S0):
    """q, k: [T][dk]; v: [T][dv]; decay, beta: [T]; S0: [dk][dv].  Returns (O [T][dv], S)."""
    S = S0.clone()
    out = []
    for t in range(q.shape[0]):
        S = S * decay[t]
        u = (v[t] - S.T @ k[t]) * beta[t]
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out), S


def chunk_prepare(q, k, v, decay, beta):
    """The state-independent part of one chunk: (Wv, Wk, P, g)."""
    g = torch.cumsum(torch.log(decay.clamp_min(1e-30)), 0)
    D = torch.exp(g[:, None] - g[None, :])
    C = q.shape[0]
    low = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
    A = torch.where(low, beta[:, None] * D * (k @ k.T), torch.zeros(()))
    Wv = beta[:, None] * v
    Wk = (beta * torch.exp(g))[:, None] * k
    for t in range(C):                      # forward substitution, row by row
        Wv[t] = Wv[t] - A[t, :t] @ Wv[:t]
        Wk[t] = Wk[t] - A[t, :t] @ Wk[:t]
    P = torch.where(low | torch.eye(C, dtype=torch.bool), D * (q @ k.T), torch.zeros(()))
    return Wv, Wk, P, g


def chunk_apply(q, k, Wv, Wk, P, g, S0):
    """The state-dependent part: (O, S1)."""
    U = Wv - Wk @ S0
    O = torch.exp(g)[:, None] * (q @ S0) + P @ U
    S1 = torch.exp(g[-1]) * S0 + (torch.exp(g[-1] - g)[:, None] * k).T @ U
    return O, S1


def scan_chunked(q, k, v, decay, beta, S0, chunk: int = 64):
    S = S0.clone()
    outs = []
    for t0 in range(0, q.shape[0], chunk):
        sl = slice(t0, t0 + chunk)
        Wv, Wk, P, g = chunk_prepare(q[sl], k[sl], v[sl], decay[sl], beta[sl])
        O, S = chunk_apply(q[sl], k[sl], Wv, Wk, P, g, S)
        outs.append(O)
    return torch.cat(outs), S
