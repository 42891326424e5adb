"""fp32 oracle of the forward pass in plain PyTorch.

Single sequence, every intermediate fp32, weights used at their stored precision (bf16 dense,
q4 experts dequantised to fp32).  It is the numerical reference for every kernel test and for
the engine's logits (the role of the reference's src/ref/ref_model.cpp; the math follows
docs/MODEL.md:59-231), and it additionally implements the MTP head, which the reference's CPU
model does not have.

The functions are written per component (``hc_mix``, ``combine``, ``gdn``, ``qsa``, ``moe``,
``ple``) so kernel tests can call them on their own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .config import ModelConfig
from .ngram import NgramHasher
from .ple import PleTable
from .quant import dequantize_q4
from .weights import Weights


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + eps).float()


def gemma_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return rms(x, eps) * w


def rope_tables(cfg: ModelConfig, pos: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    half = cfg.rope_dim // 2
    inv = torch.pow(torch.tensor(cfg.rope_theta, dtype=torch.float64),
                    -2.0 * torch.arange(half, dtype=torch.float64) / cfg.rope_dim)
    ang = pos.double().unsqueeze(-1) * inv
    return torch.cos(ang).float(), torch.sin(ang).float()


def rope(cfg: ModelConfig, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """NeoX rotation of the first rope_dim dims; x [T, ..., D], pos [T]."""
    half = cfg.rope_dim // 2
    c, s = rope_tables(cfg, pos.cpu())
    c, s = c.to(x.device), s.to(x.device)
    while c.dim() < x.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    x1, x2 = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = x1 * c - x2 * s
    out[..., half:2 * half] = x2 * c + x1 * s
    return out


@dataclass
class QsaCache:
    k: List[torch.Tensor] = field(default_factory=list)      # per token [kv_heads*head_dim]
    v: List[torch.Tensor] = field(default_factory=list)
    raw_k: List[torch.Tensor] = field(default_factory=list)  # per token [idx_dim]
    ck: List[torch.Tensor] = field(default_factory=list)     # per complete group [idx_dim]


@dataclass
class RefState:
    n_tokens: int = 0
    tokens: List[int] = field(default_factory=list)
    gdn_conv: Optional[torch.Tensor] = None   # [n_gdn, conv-1, gdn_qkv]
    gdn_S: Optional[torch.Tensor] = None      # [n_gdn, v_heads, dim(k), dim(v)]
    qsa: List[QsaCache] = field(default_factory=list)
    ple_conv: Optional[torch.Tensor] = None   # [(conv-1)*dilation, hch]
    # MTP
    mtp_qsa: Optional[QsaCache] = None
    mtp_n: int = 0
    last_hidden: Optional[torch.Tensor] = None   # backbone pre-final-mixer X of the last token [hch]


class RefModel:
    def __init__(self, cfg: ModelConfig, weights: Weights, ple_table: Optional[PleTable] = None, device="cpu"):
        self.cfg, self.w, self.table, self.dev = cfg, weights, ple_table, torch.device(device)
        self.hasher = NgramHasher(cfg)
        self.dump_layers: Optional[List[torch.Tensor]] = None
        self._f32: Dict[str, torch.Tensor] = {}

    # ---- helpers
    def W(self, name: str) -> torch.Tensor:
        t = self._f32.get(name)
        if t is None:
            t = self.w[name].to(self.dev).float()
            if len(self._f32) > 64:
                self._f32.clear()
            self._f32[name] = t
        return t

    def new_state(self) -> RefState:
        c = self.cfg
        st = RefState()
        st.gdn_conv = torch.zeros(c.n_gdn, c.gdn_conv - 1, c.gdn_qkv, device=self.dev)
        st.gdn_S = torch.zeros(c.n_gdn, c.gdn_v_heads, c.gdn_dim, c.gdn_dim, device=self.dev)
        st.qsa = [QsaCache() for _ in range(c.n_qsa)]
        st.ple_conv = torch.zeros((c.ple_conv - 1) * c.ple_dilation, c.hch, device=self.dev)
        st.mtp_qsa = QsaCache()
        return st

    # ---- hyper-connections
    def hc_mix(self, prefix: str, X: torch.Tensor, inject: bool = True):
        c = self.cfg
        T = X.shape[0]
        xn = gemma_norm(X.view(T, c.hc, c.hidden), self.W(prefix + "hc_norm.weight").view(c.hc, c.hidden), c.eps)
        xn = xn.reshape(T, c.hch)
        d = xn @ self.W(prefix + "input_mix_weight_down.weight").T
        inj = xn @ self.W(prefix + "block_inject_weight.weight").T if inject else None
        u = F.silu(d / c.hc)
        g = torch.sigmoid(u @ self.W(prefix + "input_mix_weight_up.weight").T)
        block_in = (g * xn).view(T, c.hc, c.hidden).mean(1)
        return block_in, inj

    def combine(self, X, block_out, inj):
        c = self.cfg
        w = 2.0 * torch.sigmoid(inj / c.hc)                       # [T, hc]
        return X + (w.unsqueeze(-1) * block_out.unsqueeze(1)).reshape(X.shape[0], c.hch)

    # ---- PLE
    def ple_embed(self, st: RefState, tokens: List[int]) -> torch.Tensor:
        ids = self.hasher.ids_for(st.tokens[-2:], tokens)
        return self.table.gather(ids).to(self.dev)

    def ple(self, st: RefState, X: torch.Tensor, tokens: List[int], e: Optional[torch.Tensor] = None):
        c = self.cfg
        p = f"layers.{c.ple_layer}.ple."
        T = X.shape[0]
        if e is None:
            e = self.ple_embed(st, tokens)
        key = e @ self.W(p + "key_proj.weight").T                   # [T, hch]
        val = e @ self.W(p + "value_proj.weight").T                 # [T, H]
        kn = gemma_norm(key.view(T, c.hc, c.hidden), self.W(p + "norm_key.weight").view(c.hc, c.hidden), c.eps)
        qn = gemma_norm(X.view(T, c.hc, c.hidden), self.W(p + "norm_query.weight").view(c.hc, c.hidden), c.eps)
        gs = (kn * qn).sum(-1) / math.sqrt(c.hidden)                # [T, hc]
        mag = torch.sqrt(gs.abs().clamp_min(1e-6))
        gate = torch.sigmoid(torch.sign(gs) * mag)
        gv = gate.unsqueeze(-1) * val.unsqueeze(1)                  # [T, hc, H]
        nc = gemma_norm(gv, self.W(p + "norm_conv.weight").view(c.hc, c.hidden), c.eps).reshape(T, c.hch)
        hist = (c.ple_conv - 1) * c.ple_dilation
        seq = torch.cat([st.ple_conv, nc], 0)                       # [hist+T, hch]
        cw = self.W(p + "conv1d.weight").view(c.hch, c.ple_conv)
        acc = torch.zeros(T, c.hch, device=self.dev)
        for k in range(c.ple_conv):
            acc += cw[:, k] * seq[k * c.ple_dilation: k * c.ple_dilation + T]
        st.ple_conv = seq[-hist:].clone()
        return X + gv.reshape(T, c.hch) + F.silu(acc)

    # ---- GDN
    def gdn(self, st: RefState, L: int, x: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        p = f"layers.{L}.linear_attn."
        gi = c.gdn_index(L)
        T = x.shape[0]
        qkv = x @ self.W(p + "in_proj_qkv.weight").T
        z = x @ self.W(p + "in_proj_z.weight").T
        b = x @ self.W(p + "in_proj_b.weight").T
        a = x @ self.W(p + "in_proj_a.weight").T
        cw = self.W(p + "conv1d.weight").view(c.gdn_qkv, c.gdn_conv)
        seq = torch.cat([st.gdn_conv[gi], qkv], 0)
        acc = torch.zeros(T, c.gdn_qkv, device=self.dev)
        for k in range(c.gdn_conv):
            acc += cw[:, k] * seq[k:k + T]
        st.gdn_conv[gi] = seq[-(c.gdn_conv - 1):]
        qkv = F.silu(acc)
        q = qkv[:, :c.gdn_key].view(T, c.gdn_qk_heads, c.gdn_dim)
        k = qkv[:, c.gdn_key:2 * c.gdn_key].view(T, c.gdn_qk_heads, c.gdn_dim)
        v = qkv[:, 2 * c.gdn_key:].view(T, c.gdn_v_heads, c.gdn_dim)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + c.eps) / math.sqrt(c.gdn_dim)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + c.eps)
        g = -torch.exp(self.W(p + "A_log")) * F.softplus(a + self.W(p + "dt_bias"), threshold=20.0)
        beta = torch.sigmoid(b)
        rep = c.gdn_v_heads // c.gdn_qk_heads
        kk = k.repeat_interleave(rep, dim=1)                        # [T, vh, dim]
        qq = q.repeat_interleave(rep, dim=1)
        S = st.gdn_S[gi]                                            # [vh, k, v]
        o = torch.empty(T, c.gdn_v_heads, c.gdn_dim, device=self.dev)
        for t in range(T):
            S = S * torch.exp(g[t]).view(-1, 1, 1)
            u = (v[t] - torch.einsum("hkv,hk->hv", S, kk[t])) * beta[t].unsqueeze(-1)
            S = S + kk[t].unsqueeze(-1) * u.unsqueeze(1)
            o[t] = torch.einsum("hkv,hk->hv", S, qq[t])
        st.gdn_S[gi] = S
        o = plain_norm(o, self.W(p + "norm.weight"), c.eps) * torch.sigmoid(z.view(T, c.gdn_v_heads, c.gdn_dim))
        return o.reshape(T, c.gdn_val) @ self.W(p + "out_proj.weight").T

    # ---- QSA
    def qsa_select(self, iqh_t: torch.Tensor, ck: torch.Tensor, pos: int) -> torch.Tensor:
        """Token positions attended by the query at ``pos``."""
        c = self.cfg
        nb = (pos + 1) // c.idx_ratio
        if nb <= c.idx_topk_blocks:
            return torch.arange(pos + 1, device=self.dev)
        sc = torch.relu(ck[:nb] @ iqh_t.T).sum(-1) / math.sqrt(c.idx_dim)          # [nb]
        # top-k with ties to the lowest index: stable sort of -score
        order = torch.sort(-sc, stable=True).indices[:c.idx_topk_blocks]
        sel = (order.unsqueeze(-1) * c.idx_ratio + torch.arange(c.idx_ratio, device=self.dev)).reshape(-1)
        tail = torch.arange(nb * c.idx_ratio, pos + 1, device=self.dev)
        return torch.cat([sel, tail])

    def qsa(self, cache: QsaCache, prefix: str, x: torch.Tensor, base: int) -> torch.Tensor:
        c = self.cfg
        p = prefix
        T = x.shape[0]
        qg = (x @ self.W(p + "q_proj.weight").T).view(T, c.q_heads, 2, c.head_dim)
        q, gate = qg[:, :, 0], qg[:, :, 1]
        k = (x @ self.W(p + "k_proj.weight").T).view(T, c.kv_heads, c.head_dim)
        v = (x @ self.W(p + "v_proj.weight").T).view(T, c.kv_heads, c.head_dim)
        iq = x @ self.W(p + "indexer.index_qk_proj.weight").T
        pos = torch.arange(base, base + T)
        q = rope(c, gemma_norm(q, self.W(p + "q_norm.weight"), c.eps), pos)
        k = rope(c, gemma_norm(k, self.W(p + "k_norm.weight"), c.eps), pos)
        iqh = iq[:, :c.idx_heads * c.idx_dim].view(T, c.idx_heads, c.idx_dim)
        iqh = rope(c, gemma_norm(iqh, self.W(p + "indexer.q_layernorm.weight"), c.eps), pos)
        rawk = iq[:, c.idx_heads * c.idx_dim:]
        for t in range(T):
            cache.k.append(k[t].reshape(-1))
            cache.v.append(v[t].reshape(-1))
            cache.raw_k.append(rawk[t])
            P = base + t
            if (P + 1) % c.idx_ratio == 0:
                mean = torch.stack(cache.raw_k[P + 1 - c.idx_ratio: P + 1]).mean(0)
                nk = gemma_norm(mean, self.W(p + "indexer.k_layernorm.weight"), c.eps)
                cache.ck.append(rope(c, nk.unsqueeze(0), torch.tensor([P + 1 - c.idx_ratio]))[0])
        K = torch.stack(cache.k).view(-1, c.kv_heads, c.head_dim)
        V = torch.stack(cache.v).view(-1, c.kv_heads, c.head_dim)
        CK = torch.stack(cache.ck) if cache.ck else torch.zeros(0, c.idx_dim, device=self.dev)
        rep = c.q_heads // c.kv_heads
        o = torch.empty(T, c.q_heads, c.head_dim, device=self.dev)
        for t in range(T):
            sel = self.qsa_select(iqh[t], CK, base + t)
            Ks = K[sel].repeat_interleave(rep, dim=1)               # [n, qh, D]
            Vs = V[sel].repeat_interleave(rep, dim=1)
            logit = torch.einsum("hd,nhd->hn", q[t], Ks) / math.sqrt(c.head_dim)
            w = torch.softmax(logit.double(), dim=-1).float()
            o[t] = torch.einsum("hn,nhd->hd", w, Vs)
        o = o * torch.sigmoid(gate)
        return o.reshape(T, c.q_heads * c.head_dim) @ self.W(p + "o_proj.weight").T

    # ---- MoE
    def route(self, prefix: str, x: torch.Tensor):
        c = self.cfg
        logits = x @ self.W(prefix + "gate.weight").T
        pr = torch.softmax(logits, dim=-1)
        order = torch.sort(-pr, dim=-1, stable=True).indices[:, :c.top_k]        # ties -> lowest index
        top = torch.gather(pr, 1, order)
        return order, top / top.sum(-1, keepdim=True), logits

    def expert_w(self, prefix: str, proj: str, e: int) -> torch.Tensor:
        pk = self.w[prefix + f"experts.{proj}.weight_packed"][e]
        sc = self.w[prefix + f"experts.{proj}.weight_scale"][e]
        return dequantize_q4(pk, sc, self.cfg.qgroup).to(self.dev)

    def moe(self, prefix: str, x: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        p = prefix
        T = x.shape[0]
        idx, wgt, _ = self.route(p, x)
        out = torch.zeros(T, c.hidden, device=self.dev)
        for e in torch.unique(idx).tolist():
            rows, slot = torch.nonzero(idx == e, as_tuple=True)
            xs = x[rows]
            h = F.silu(xs @ self.expert_w(p, "gate_proj", e).T) * (xs @ self.expert_w(p, "up_proj", e).T)
            y = h @ self.expert_w(p, "down_proj", e).T
            out.index_add_(0, rows, y * wgt[rows, slot].unsqueeze(-1))
        h = F.silu(x @ self.W(p + "shared_expert.gate_proj.weight").T) * (x @ self.W(p + "shared_expert.up_proj.weight").T)
        y = h @ self.W(p + "shared_expert.down_proj.weight").T
        sg = torch.sigmoid(x @ self.W(p + "shared_expert_gate.weight").T)
        return out + sg * y

    # ---- full forward
    def embed(self, tokens: List[int]) -> torch.Tensor:
        c = self.cfg
        t = torch.tensor([c.real_token(int(x)) for x in tokens], dtype=torch.long)
        e = self.w["embed_tokens.weight"][t].to(self.dev).float()
        return e

    def decoder_layer(self, st: RefState, L: int, X, pending, tokens, ple_e=None):
        c = self.cfg
        p = f"layers.{L}."
        if pending is not None:
            X = self.combine(X, *pending)
        if L == c.ple_layer and self.table is not None:
            X = self.ple(st, X, tokens, ple_e)
        a_in, a_inj = self.hc_mix(p + "attn_hyper_connection.", X)
        if c.is_qsa(L):
            a_out = self.qsa(st.qsa[c.qsa_index(L)], p + "self_attn.", a_in, st.n_tokens)
        else:
            a_out = self.gdn(st, L, a_in)
        X = self.combine(X, a_out, a_inj)
        m_in, m_inj = self.hc_mix(p + "mlp_hyper_connection.", X)
        m_out = self.moe(p + "mlp.", m_in)
        return X, (m_out, m_inj)

    @torch.no_grad()
    def forward(self, st: RefState, tokens: List[int], all_logits: bool = False, embeds: Optional[torch.Tensor] = None,
                return_hidden: bool = False):
        """Append ``tokens`` to the sequence and return logits of the last token (or all)."""
        c = self.cfg
        T = len(tokens)
        assert T > 0
        if st.gdn_S is None:
            st.__dict__.update(self.new_state().__dict__)
        e = self.embed(tokens) if embeds is None else embeds.to(self.dev).float()
        X = e.repeat(1, c.hc)
        pending = None
        if self.dump_layers is not None:
            self.dump_layers.clear()
        for L in range(c.n_layers):
            X, pending = self.decoder_layer(st, L, X, pending, tokens)
            if self.dump_layers is not None:
                self.dump_layers.append(self.combine(X, *pending).clone())
        Xf = self.combine(X, *pending)
        y, _ = self.hc_mix("hyper_connection_mixer.", Xf, inject=False)
        head = self.W("lm_head.weight")
        logits = (y if all_logits else y[-1:]) @ head.T
        st.tokens.extend(int(t) for t in tokens)
        st.n_tokens += T
        st.last_hidden = Xf
        if return_hidden:
            return logits, Xf
        return logits

    # ---- MTP head
    @torch.no_grad()
    def mtp_forward(self, st: RefState, hidden: torch.Tensor, next_tokens: List[int], base: int):
        """One MTP pass over rows: ``hidden [T, hch]`` is the pre-final-mixer state of positions
        ``base..base+T-1`` and ``next_tokens[t]`` the token at position ``base+t+1``.  Returns the
        draft logits ``[T, vocab]`` (prediction for position ``base+t+2``) and the MTP's own
        pre-final-mixer hidden, which replaces ``hidden`` in later draft steps."""
        c = self.cfg
        T = hidden.shape[0]
        hn = rms(hidden, c.eps) * (1.0 + self.W("mtp.pre_fc_norm_hidden.weight"))      # one RMS over all hch values
        en = gemma_norm(self.embed(next_tokens), self.W("mtp.pre_fc_norm_embedding.weight"), c.eps)
        fe = en @ self.W("mtp.fc_embedding.weight").T                                  # [T, H]
        fh = hn.view(T, c.hc, c.hidden) @ self.W("mtp.fc_hidden.weight").T             # [T, hc, H]
        X = (fh + fe.unsqueeze(1)).reshape(T, c.hch)
        p = "mtp.layers.0."
        a_in, a_inj = self.hc_mix(p + "attn_hyper_connection.", X)
        a_out = self.qsa(st.mtp_qsa, p + "self_attn.", a_in, base)
        X = self.combine(X, a_out, a_inj)
        m_in, m_inj = self.hc_mix(p + "mlp_hyper_connection.", X)
        m_out = self.moe(p + "mlp.", m_in)
        Xf = self.combine(X, m_out, m_inj)
        y, _ = self.hc_mix("mtp.hyper_connection_mixer.", Xf, inject=False)
        st.mtp_n = base + T
        return y @ self.W("lm_head.weight").T, Xf


def greedy_generate(model: RefModel, prompt: List[int], n_new: int):
    """Greedy continuation; returns (tokens, logits of each generated position)."""
    st = model.new_state()
    logits = model.forward(st, prompt)
    out, all_logits = [], []
    for _ in range(n_new):
        all_logits.append(logits[-1].clone())
        t = int(torch.argmax(logits[-1]))
        out.append(t)
        logits = model.forward(st, [t])
    return out, torch.stack(all_logits)
