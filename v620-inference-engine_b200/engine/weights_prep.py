"""Checkpoint-layout weights -> one rank's engine layout.

Slices every tensor for tensor parallelism (attention heads, GDN heads, shared-expert columns,
vocabulary rows), expert parallelism (a contiguous block of routed experts) and the hidden-dim
sharded residual (hyper-connection mixers, PLE), concatenates projections that share an input
into one matrix, folds ``1 + w`` into the Gemma-norm weights and re-orders the q4 nibbles into
the engine order (role of the reference's src/engine/weights.hip:230-418 and
src/engine/weight_convert.cpp; bf16 stays bf16 here instead of becoming fp16).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..models.config import ModelConfig, ShardConfig
from ..models.quant import to_engine_order
from ..models.weights import Weights

T = torch.Tensor


def _dev(t: T, device) -> T:
    return t.to(device, non_blocking=True)


def prep_hc(w: Weights, prefix: str, sc: ShardConfig, inject: bool, device) -> Dict[str, T]:
    c = sc.cfg
    cols = sc.cols()
    norm = _dev(w[prefix + "hc_norm.weight"], device).float().view(c.hc, c.hidden)[:, cols]
    down = _dev(w[prefix + "input_mix_weight_down.weight"], device).view(c.hc_rank, c.hc, c.hidden)[:, :, cols]
    rows = [down]
    if inject:
        rows.append(_dev(w[prefix + "block_inject_weight.weight"], device).view(c.hc, c.hc, c.hidden)[:, :, cols])
    up = _dev(w[prefix + "input_mix_weight_up.weight"], device).view(c.hc, c.hidden, c.hc_rank)[:, cols, :]
    return {
        "w1": (1.0 + norm).contiguous(),
        "Wd": torch.cat(rows, 0).to(torch.bfloat16).contiguous(),            # [R+n_inj][hc][SH]
        "Wu": up.permute(1, 0, 2).to(torch.bfloat16).contiguous(),           # [SH][hc][R]
        "n_inj": c.hc if inject else 0,
    }


def prep_gdn(w: Weights, p: str, sc: ShardConfig, device) -> Dict[str, T]:
    c, r = sc.cfg, sc.rank
    D = c.gdn_dim
    kq = slice(r * sc.gdn_kl * D, (r + 1) * sc.gdn_kl * D)
    vv = slice(r * sc.gdn_vl * D, (r + 1) * sc.gdn_vl * D)
    vh = slice(r * sc.gdn_vl, (r + 1) * sc.gdn_vl)
    qkv = _dev(w[p + "in_proj_qkv.weight"], device)
    q, k, v = qkv[:c.gdn_key], qkv[c.gdn_key:2 * c.gdn_key], qkv[2 * c.gdn_key:]
    z = _dev(w[p + "in_proj_z.weight"], device)
    b = _dev(w[p + "in_proj_b.weight"], device)
    a = _dev(w[p + "in_proj_a.weight"], device)
    cw = _dev(w[p + "conv1d.weight"], device).float().view(c.gdn_qkv, c.gdn_conv)
    cq, ck, cv = cw[:c.gdn_key], cw[c.gdn_key:2 * c.gdn_key], cw[2 * c.gdn_key:]
    return {
        "Wproj": torch.cat([q[kq], k[kq], v[vv], z[vv], b[vh], a[vh]], 0).to(torch.bfloat16).contiguous(),
        "Wout": _dev(w[p + "out_proj.weight"], device)[:, vv].to(torch.bfloat16).contiguous(),
        "cw": torch.cat([cq[kq], ck[kq], cv[vv]], 0).contiguous(),
        "A_log": _dev(w[p + "A_log"], device).float()[vh].contiguous(),
        "dt_bias": _dev(w[p + "dt_bias"], device).float()[vh].contiguous(),
        "gdn_norm": _dev(w[p + "norm.weight"], device).float().contiguous(),
    }


def prep_qsa(w: Weights, p: str, sc: ShardConfig, device) -> Dict[str, T]:
    c, r = sc.cfg, sc.rank
    D = c.head_dim
    qrows = slice(r * sc.qh_l * 2 * D, (r + 1) * sc.qh_l * 2 * D)
    kvrows = slice(sc.kv_head0 * D, (sc.kv_head0 + sc.kvh_l) * D)
    orows = slice(r * sc.qh_l * D, (r + 1) * sc.qh_l * D)
    return {
        "Wproj": torch.cat([_dev(w[p + "q_proj.weight"], device)[qrows], _dev(w[p + "k_proj.weight"], device)[kvrows],
                            _dev(w[p + "v_proj.weight"], device)[kvrows],
                            _dev(w[p + "indexer.index_qk_proj.weight"], device)], 0).to(torch.bfloat16).contiguous(),
        "Wout": _dev(w[p + "o_proj.weight"], device)[:, orows].to(torch.bfloat16).contiguous(),
        "qn1": (1.0 + _dev(w[p + "q_norm.weight"], device).float()).contiguous(),
        "kn1": (1.0 + _dev(w[p + "k_norm.weight"], device).float()).contiguous(),
        "iqn1": (1.0 + _dev(w[p + "indexer.q_layernorm.weight"], device).float()).contiguous(),
        "ikn1": (1.0 + _dev(w[p + "indexer.k_layernorm.weight"], device).float()).contiguous(),
    }


def prep_moe(w: Weights, p: str, sc: ShardConfig, device) -> Dict[str, T]:
    c, r = sc.cfg, sc.rank
    sf = slice(r * sc.sffn_l, (r + 1) * sc.sffn_l)
    ex = slice(r * sc.exp_l, (r + 1) * sc.exp_l)
    out = {
        "Wrs": torch.cat([_dev(w[p + "gate.weight"], device), _dev(w[p + "shared_expert_gate.weight"], device),
                          _dev(w[p + "shared_expert.gate_proj.weight"], device)[sf],
                          _dev(w[p + "shared_expert.up_proj.weight"], device)[sf]], 0).to(torch.bfloat16).contiguous(),
        "Wsd": _dev(w[p + "shared_expert.down_proj.weight"], device)[:, sf].to(torch.bfloat16).contiguous(),
    }
    g = _dev(w[p + "experts.gate_proj.weight_packed"][ex], device)
    u = _dev(w[p + "experts.up_proj.weight_packed"][ex], device)
    out["w13"] = to_engine_order(torch.cat([g, u], 1)).contiguous()
    out["s13"] = torch.cat([_dev(w[p + "experts.gate_proj.weight_scale"][ex], device),
                            _dev(w[p + "experts.up_proj.weight_scale"][ex], device)], 1).to(torch.bfloat16).contiguous()
    out["w2"] = to_engine_order(_dev(w[p + "experts.down_proj.weight_packed"][ex], device)).contiguous()
    out["s2"] = _dev(w[p + "experts.down_proj.weight_scale"][ex], device).to(torch.bfloat16).contiguous()
    return out


def prep_layer(cfg: ModelConfig, w: Weights, L: int, sc: ShardConfig, device, prefix: Optional[str] = None,
               qsa: Optional[bool] = None) -> Dict[str, object]:
    p = prefix if prefix is not None else f"layers.{L}."
    qsa = cfg.is_qsa(L) if qsa is None else qsa
    out: Dict[str, object] = {"is_qsa": qsa}
    out["attn_hc"] = prep_hc(w, p + "attn_hyper_connection.", sc, True, device)
    out["mlp_hc"] = prep_hc(w, p + "mlp_hyper_connection.", sc, True, device)
    out.update(prep_qsa(w, p + "self_attn.", sc, device) if qsa else prep_gdn(w, p + "linear_attn.", sc, device))
    out.update(prep_moe(w, p + "mlp.", sc, device))
    return out


def prep_ple(cfg: ModelConfig, w: Weights, sc: ShardConfig, device) -> Dict[str, T]:
    c = cfg
    p = f"layers.{c.ple_layer}.ple."
    cols = sc.cols()
    key = _dev(w[p + "key_proj.weight"], device).view(c.hc, c.hidden, c.hidden)[:, cols, :].reshape(-1, c.hidden)
    val = _dev(w[p + "value_proj.weight"], device)[cols]

    def n1(name):
        return (1.0 + _dev(w[p + name], device).float().view(c.hc, c.hidden)[:, cols]).contiguous()
    cw = _dev(w[p + "conv1d.weight"], device).float().view(c.hc, c.hidden, c.ple_conv)[:, cols, :]
    return {
        "Wkv": torch.cat([key, val], 0).to(torch.bfloat16).contiguous(),
        "nk1": n1("norm_key.weight"), "nq1": n1("norm_query.weight"), "nc1": n1("norm_conv.weight"),
        "cw": cw.reshape(-1, c.ple_conv).contiguous(),
    }


def prep_globals(cfg: ModelConfig, w: Weights, sc: ShardConfig, device) -> Dict[str, object]:
    r = sc.rank
    vs = slice(r * sc.vocab_l, (r + 1) * sc.vocab_l)
    return {
        "embed": _dev(w["embed_tokens.weight"], device).to(torch.bfloat16).contiguous(),
        "lm_head": _dev(w["lm_head.weight"], device)[vs].to(torch.bfloat16).contiguous(),
        "final_hc": prep_hc(w, "hyper_connection_mixer.", sc, False, device),
    }
