"""Weight naming, synthesis and checkpoint loading.

Tensor names follow the checkpoint (reference docs/MODEL.md, names without the
``model.language_model.`` prefix) with one change: the routed experts of a layer are stacked
into one tensor per projection (``layers.L.mlp.experts.gate_proj.weight_packed [E, ffn, H/8]``
instead of ``experts.E.gate_proj…``), which is how the engine stores them anyway.

Everything dense is bf16; routed experts are q4 (int4 g128, checkpoint nibble order, bf16
scales).  ``synth_weights`` draws N(0, std) weights from a seed — used by the oracle slice,
the tests and the benchmarks (no checkpoint is available offline) — and ``load_checkpoint``
reads the real safetensors files.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterable, Optional

import torch

from .config import ModelConfig
from .quant import quantize_q4, random_q4

Weights = Dict[str, torch.Tensor]


def hc_names(prefix: str, inject: bool = True):
    n = [prefix + "hc_norm.weight", prefix + "input_mix_weight_down.weight", prefix + "input_mix_weight_up.weight"]
    if inject:
        n.append(prefix + "block_inject_weight.weight")
    return n


def layer_shapes(cfg: ModelConfig, L: int, prefix: Optional[str] = None, qsa: Optional[bool] = None) -> Dict[str, tuple]:
    """Name -> shape of every dense tensor of decoder layer ``L`` (experts excluded)."""
    c = cfg
    p = prefix if prefix is not None else f"layers.{L}."
    qsa = c.is_qsa(L) if qsa is None else qsa
    s: Dict[str, tuple] = {}
    for hc in ("attn_hyper_connection.", "mlp_hyper_connection."):
        s[p + hc + "hc_norm.weight"] = (c.hch,)
        s[p + hc + "input_mix_weight_down.weight"] = (c.hc_rank, c.hch)
        s[p + hc + "input_mix_weight_up.weight"] = (c.hch, c.hc_rank)
        s[p + hc + "block_inject_weight.weight"] = (c.hc, c.hch)
    if qsa:
        a = p + "self_attn."
        s[a + "q_proj.weight"] = (c.q_heads * 2 * c.head_dim, c.hidden)
        s[a + "k_proj.weight"] = (c.kv_heads * c.head_dim, c.hidden)
        s[a + "v_proj.weight"] = (c.kv_heads * c.head_dim, c.hidden)
        s[a + "q_norm.weight"] = (c.head_dim,)
        s[a + "k_norm.weight"] = (c.head_dim,)
        s[a + "o_proj.weight"] = (c.hidden, c.q_heads * c.head_dim)
        s[a + "indexer.index_qk_proj.weight"] = ((c.idx_heads + 1) * c.idx_dim, c.hidden)
        s[a + "indexer.q_layernorm.weight"] = (c.idx_dim,)
        s[a + "indexer.k_layernorm.weight"] = (c.idx_dim,)
    else:
        a = p + "linear_attn."
        s[a + "in_proj_qkv.weight"] = (c.gdn_qkv, c.hidden)
        s[a + "in_proj_z.weight"] = (c.gdn_val, c.hidden)
        s[a + "in_proj_b.weight"] = (c.gdn_v_heads, c.hidden)
        s[a + "in_proj_a.weight"] = (c.gdn_v_heads, c.hidden)
        s[a + "conv1d.weight"] = (c.gdn_qkv, 1, c.gdn_conv)
        s[a + "A_log"] = (c.gdn_v_heads,)
        s[a + "dt_bias"] = (c.gdn_v_heads,)
        s[a + "norm.weight"] = (c.gdn_dim,)
        s[a + "out_proj.weight"] = (c.hidden, c.gdn_val)
    m = p + "mlp."
    s[m + "gate.weight"] = (c.n_experts, c.hidden)
    s[m + "shared_expert.gate_proj.weight"] = (c.ffn, c.hidden)
    s[m + "shared_expert.up_proj.weight"] = (c.ffn, c.hidden)
    s[m + "shared_expert.down_proj.weight"] = (c.hidden, c.ffn)
    s[m + "shared_expert_gate.weight"] = (1, c.hidden)
    if L == c.ple_layer and prefix is None:
        e = p + "ple."
        s[e + "key_proj.weight"] = (c.hch, c.hidden)
        s[e + "value_proj.weight"] = (c.hidden, c.hidden)
        s[e + "norm_key.weight"] = (c.hch,)
        s[e + "norm_query.weight"] = (c.hch,)
        s[e + "norm_conv.weight"] = (c.hch,)
        s[e + "conv1d.weight"] = (c.hch, 1, c.ple_conv)
    return s


def global_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    c = cfg
    s = {
        "embed_tokens.weight": (c.vocab, c.hidden),
        "lm_head.weight": (c.vocab, c.hidden),
        "hyper_connection_mixer.hc_norm.weight": (c.hch,),
        "hyper_connection_mixer.input_mix_weight_down.weight": (c.hc_rank, c.hch),
        "hyper_connection_mixer.input_mix_weight_up.weight": (c.hch, c.hc_rank),
    }
    if c.mtp:
        s.update({
            "mtp.fc_hidden.weight": (c.hidden, c.hidden),
            "mtp.fc_embedding.weight": (c.hidden, c.hidden),
            "mtp.pre_fc_norm_hidden.weight": (c.hch,),
            "mtp.pre_fc_norm_embedding.weight": (c.hidden,),
            "mtp.hyper_connection_mixer.hc_norm.weight": (c.hch,),
            "mtp.hyper_connection_mixer.input_mix_weight_down.weight": (c.hc_rank, c.hch),
            "mtp.hyper_connection_mixer.input_mix_weight_up.weight": (c.hch, c.hc_rank),
        })
    return s


def _dense(name: str, shape: tuple, gen: torch.Generator, std: float, device) -> torch.Tensor:
    if name.endswith("A_log"):
        t = torch.rand(shape, generator=gen, device=device) * 2.0 - 0.5
    elif name.endswith("dt_bias"):
        t = torch.randn(shape, generator=gen, device=device) * 0.5
    elif "norm" in name or "layernorm" in name:
        t = torch.randn(shape, generator=gen, device=device) * 0.1
        if name.endswith("linear_attn.norm.weight"):
            t = t + 1.0          # plain norm multiplies by w (not 1+w)
    elif "conv1d" in name:
        t = torch.randn(shape, generator=gen, device=device) * 0.3
    else:
        t = torch.randn(shape, generator=gen, device=device) * std
    return t.to(torch.bfloat16)


def synth_experts(cfg: ModelConfig, gen: torch.Generator, std: float, device, exact: bool, prefix: str,
                  experts: Optional[Iterable[int]] = None) -> Weights:
    """q4 routed experts of one layer.  ``exact``: draw N(0,std) bf16 weights and quantise them
    (oracle slice, tests); else draw random nibbles directly (full-size synthetic model)."""
    c = cfg
    ne = c.n_experts if experts is None else len(list(experts))
    out: Weights = {}
    for proj, (o, i) in (("gate_proj", (c.ffn, c.hidden)), ("up_proj", (c.ffn, c.hidden)),
                         ("down_proj", (c.hidden, c.ffn))):
        if exact:
            w = (torch.randn((ne * o, i), generator=gen, device=device) * std).to(torch.bfloat16)
            pk, sc = quantize_q4(w, c.qgroup, torch.bfloat16)
        else:
            pk, sc = random_q4(ne * o, i, std=std, generator=gen, device=device)
        out[prefix + f"experts.{proj}.weight_packed"] = pk.reshape(ne, o, i // 8)
        out[prefix + f"experts.{proj}.weight_scale"] = sc.reshape(ne, o, i // c.qgroup)
    return out


def synth_layer(cfg: ModelConfig, L: int, seed: int = 0, std: float = 0.02, device="cpu", exact: bool = True,
                prefix: Optional[str] = None, qsa: Optional[bool] = None) -> Weights:
    gen = torch.Generator(device=device).manual_seed(seed * 100003 + (L + 1) * 7919 + (0 if prefix is None else 1))
    w: Weights = {}
    for name, shape in layer_shapes(cfg, L, prefix, qsa).items():
        w[name] = _dense(name, shape, gen, std, device)
    p = prefix if prefix is not None else f"layers.{L}."
    w.update(synth_experts(cfg, gen, std, device, exact, p + "mlp."))
    return w


def synth_globals(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu") -> Weights:
    gen = torch.Generator(device=device).manual_seed(seed * 100003 + 17)
    return {n: _dense(n, s, gen, std, device) for n, s in global_shapes(cfg).items()}


def synth_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu", exact: bool = True) -> Weights:
    """All weights of the model.  Only for models that fit in host memory (slices, tiny models);
    the engine synthesises full-size models layer by layer on the device."""
    w = synth_globals(cfg, seed, std, device)
    for L in range(cfg.n_layers):
        w.update(synth_layer(cfg, L, seed, std, device, exact))
    if cfg.mtp:
        w.update(synth_layer(cfg, cfg.n_layers, seed, std, device, exact, prefix="mtp.layers.0.", qsa=True))
    return w


PREFIX = "model.language_model."


def load_checkpoint(cfg: ModelConfig, model_dir: str, layers: Optional[Iterable[int]] = None) -> Weights:
    """Read a real checkpoint (safetensors shards; experts listed one by one, MTP experts bf16 with a
    fused gate_up_proj) into the stacked naming above.  MTP experts are quantised to q4 at load
    (reference src/engine/weights.hip:352-369, weight_convert.cpp:73-90)."""
    from safetensors import safe_open
    want = None if layers is None else {f"layers.{i}." for i in layers}
    raw: Weights = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        with safe_open(path, "pt") as f:
            for k in f.keys():
                n = k[len(PREFIX):] if k.startswith(PREFIX) else k
                if want is not None and n.startswith("layers.") and not any(n.startswith(p) for p in want):
                    continue
                raw[n] = f.get_tensor(k)
    out: Weights = {}
    stacks: Dict[str, Dict[int, torch.Tensor]] = {}
    for n, t in raw.items():
        if ".mlp.experts." in n and n.split(".mlp.experts.")[1].split(".")[0].isdigit():
            head, tail = n.split(".mlp.experts.")
            e, rest = tail.split(".", 1)
            stacks.setdefault(head + ".mlp.experts." + rest, {})[int(e)] = t
        else:
            out[n] = t
    for n, d in stacks.items():
        out[n] = torch.stack([d[i] for i in range(len(d))])
    # MTP: bf16 fused experts -> q4
    k = "mtp.layers.0.mlp.experts.gate_up_proj"
    if k in out:
        gu = out.pop(k)                                      # [E, 2*ffn, H], gate rows first
        dn = out.pop("mtp.layers.0.mlp.experts.down_proj")   # [E, H, ffn]
        E = gu.shape[0]
        for proj, w in (("gate_proj", gu[:, :cfg.ffn]), ("up_proj", gu[:, cfg.ffn:]), ("down_proj", dn)):
            pk, sc = quantize_q4(w.reshape(-1, w.shape[-1]).contiguous(), cfg.qgroup, torch.bfloat16)
            out[f"mtp.layers.0.mlp.experts.{proj}.weight_packed"] = pk.reshape(E, w.shape[1], -1)
            out[f"mtp.layers.0.mlp.experts.{proj}.weight_scale"] = sc.reshape(E, w.shape[1], -1)
    return out
