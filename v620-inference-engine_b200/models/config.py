"""Model shapes and per-rank shard shapes.

The served model is fixed (reference: src/core/config.hpp:11-81 holds every shape as a
compile-time constant and src/core/shard.hpp:12-37 the 4-rank shard shapes).  Here the
shapes live in a frozen dataclass so that the same code runs the full 180B model, the
two-layer fp32 oracle slice and the tiny models of the unit tests, and the rank count is a
runtime value validated to be 1, 2, 4 or 8.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Tuple


@dataclass(frozen=True)
class ModelConfig:
    # trunk
    hidden: int = 2560
    hc: int = 4                      # hyper-connection streams
    hc_rank: int = 320               # low rank of the mixer
    n_layers: int = 48
    vocab: int = 248320
    eos: int = 248044
    eps: float = 1e-6
    image_pad: int = 248056
    video_pad: int = 248057
    # layer i is QSA when i % qsa_every == qsa_every-1 unless layer_types is given
    qsa_every: int = 4
    layer_types: Tuple[str, ...] = ()   # optional explicit ("gdn"|"qsa") per layer
    # QSA
    q_heads: int = 24
    kv_heads: int = 2
    head_dim: int = 256
    rope_dim: int = 64
    rope_theta: float = 1e7
    idx_heads: int = 4
    idx_dim: int = 128
    idx_budget: int = 2048           # tokens
    idx_ratio: int = 4               # tokens per compressed group
    # GDN
    gdn_qk_heads: int = 16
    gdn_v_heads: int = 48
    gdn_dim: int = 128
    gdn_conv: int = 4
    gdn_ring: int = 8
    # MoE
    n_experts: int = 512
    top_k: int = 10
    ffn: int = 640
    qgroup: int = 128
    # PLE
    ple_layer: int = 1
    ngram: int = 3
    ngram_heads: int = 16
    ple_conv: int = 4
    ple_dilation: int = 3
    ple_ring: int = 16
    ngram_vocab_base: int = 20_000_000
    ple_seed: int = 1234
    # MTP
    mtp: bool = True

    # ---- derived
    @property
    def hch(self) -> int:
        return self.hc * self.hidden

    @property
    def hc_down(self) -> int:          # low-rank rows + inject rows
        return self.hc_rank + self.hc

    @property
    def idx_topk_blocks(self) -> int:
        return self.idx_budget // self.idx_ratio

    @property
    def gdn_key(self) -> int:
        return self.gdn_qk_heads * self.gdn_dim

    @property
    def gdn_val(self) -> int:
        return self.gdn_v_heads * self.gdn_dim

    @property
    def gdn_qkv(self) -> int:
        return 2 * self.gdn_key + self.gdn_val

    @property
    def ngram_dim(self) -> int:
        return self.hidden // self.ngram_heads

    def is_qsa(self, layer: int) -> bool:
        if self.layer_types:
            return self.layer_types[layer] == "qsa"
        return layer % self.qsa_every == self.qsa_every - 1

    @property
    def qsa_layers(self) -> Tuple[int, ...]:
        return tuple(i for i in range(self.n_layers) if self.is_qsa(i))

    @property
    def gdn_layers(self) -> Tuple[int, ...]:
        return tuple(i for i in range(self.n_layers) if not self.is_qsa(i))

    @property
    def n_qsa(self) -> int:
        return len(self.qsa_layers)

    @property
    def n_gdn(self) -> int:
        return len(self.gdn_layers)

    def qsa_index(self, layer: int) -> int:
        return self.qsa_layers.index(layer)

    def gdn_index(self, layer: int) -> int:
        return self.gdn_layers.index(layer)

    def real_token(self, t: int) -> int:
        """Vision tokens are negative ids inside the engine (odd = image, even = video);
        the n-gram table sees the pad token instead (reference: config.hpp:24-27)."""
        if t >= 0:
            return t
        return self.image_pad if ((-t) & 1) else self.video_pad

    def validate(self) -> None:
        assert self.hidden % self.ngram_heads == 0
        assert self.q_heads % self.kv_heads == 0
        assert self.gdn_v_heads % self.gdn_qk_heads == 0
        assert self.hidden % self.qgroup == 0 and self.ffn % self.qgroup == 0
        assert self.idx_budget % self.idx_ratio == 0
        assert 0 <= self.eos < self.vocab
        if self.layer_types:
            assert len(self.layer_types) == self.n_layers

    # ---- factories
    @staticmethod
    def full() -> "ModelConfig":
        return ModelConfig()

    @staticmethod
    def slice2() -> "ModelConfig":
        """The two-layer oracle slice: one GDN layer then one QSA layer at the full per-layer
        shapes, PLE on layer 1, no MTP."""
        return ModelConfig(n_layers=2, layer_types=("gdn", "qsa"), mtp=False)

    @staticmethod
    def tiny(**kw) -> "ModelConfig":
        """A small model for unit tests.  Head dims stay at their real values because the
        kernels specialise on them; widths, head counts, experts and vocab shrink."""
        base = dict(
            hidden=256, hc_rank=32, n_layers=4, vocab=1024, eos=1000, image_pad=1001, video_pad=1002,
            q_heads=8, kv_heads=2, idx_heads=4, idx_budget=64, gdn_qk_heads=8, gdn_v_heads=16,
            n_experts=32, top_k=4, ffn=128, ngram_vocab_base=2000,
        )
        base.update(kw)
        c = ModelConfig(**base)
        c.validate()
        return c

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self))

    @staticmethod
    def from_json(s: str) -> "ModelConfig":
        d = json.loads(s)
        d["layer_types"] = tuple(d.get("layer_types", ()))
        return ModelConfig(**d)


def check_hf_config(cfg: ModelConfig, model_dir: str) -> None:
    """Verify a checkpoint's config.json against the shapes (reference: config.cpp:9-64)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    t = j.get("text_config", j)
    want = {
        "hidden_size": cfg.hidden, "num_hidden_layers": cfg.n_layers, "vocab_size": cfg.vocab,
        "num_attention_heads": cfg.q_heads, "num_key_value_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
        "num_experts": cfg.n_experts, "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.ffn,
        "hc_count": cfg.hc, "hc_lowrank": cfg.hc_rank,
        "linear_num_key_heads": cfg.gdn_qk_heads, "linear_num_value_heads": cfg.gdn_v_heads,
        "linear_key_head_dim": cfg.gdn_dim, "linear_conv_kernel_dim": cfg.gdn_conv,
    }
    bad = [f"{k}: checkpoint {t[k]} != engine {v}" for k, v in want.items() if k in t and t[k] != v]
    if bad:
        raise ValueError("config.json does not describe the served model: " + "; ".join(bad))


VALID_RANKS = (1, 2, 4, 8)


@dataclass(frozen=True)
class ShardConfig:
    """Per-rank shapes for ``ranks``-way tensor + expert parallelism with the residual
    stream sharded along the hidden dim (reference: src/core/shard.hpp:12-37 for 4 ranks)."""
    cfg: ModelConfig
    ranks: int = 1
    rank: int = 0

    def __post_init__(self):
        c, r = self.cfg, self.ranks
        if r not in VALID_RANKS:
            raise ValueError(f"ranks must be one of {VALID_RANKS}, got {r}")
        if not (0 <= self.rank < r):
            raise ValueError("rank out of range")
        for name, v in (("hidden", c.hidden), ("q_heads", c.q_heads), ("gdn_v_heads", c.gdn_v_heads),
                        ("gdn_qk_heads", c.gdn_qk_heads), ("n_experts", c.n_experts), ("ffn", c.ffn),
                        ("vocab", c.vocab)):
            if v % r:
                raise ValueError(f"{name}={v} is not divisible by ranks={r}")

    # residual
    @property
    def sh(self) -> int:            # residual columns per rank per stream
        return self.cfg.hidden // self.ranks

    @property
    def xw(self) -> int:            # a rank's slice of a multi-stream row
        return self.cfg.hc * self.sh

    @property
    def hc_send(self) -> int:       # ssq[hc] + down partials [hc][hc_down]
        return self.cfg.hc + self.cfg.hc * self.cfg.hc_down

    # GDN
    @property
    def gdn_vl(self) -> int:
        return self.cfg.gdn_v_heads // self.ranks

    @property
    def gdn_kl(self) -> int:
        return self.cfg.gdn_qk_heads // self.ranks

    @property
    def gdn_qkv_l(self) -> int:
        return (2 * self.gdn_kl + self.gdn_vl) * self.cfg.gdn_dim

    @property
    def gdn_proj_l(self) -> int:    # qkv | z | b | a
        return self.gdn_qkv_l + self.gdn_vl * self.cfg.gdn_dim + 2 * self.gdn_vl

    @property
    def gdn_state(self) -> int:     # floats per layer per sequence
        return self.gdn_vl * self.cfg.gdn_dim * self.cfg.gdn_dim

    # QSA
    @property
    def qh_l(self) -> int:
        return self.cfg.q_heads // self.ranks

    @property
    def kvh_l(self) -> int:         # KV heads stored per rank
        return max(1, self.cfg.kv_heads // self.ranks)

    @property
    def kv_replicas(self) -> int:   # ranks holding the same KV head
        return max(1, self.ranks // self.cfg.kv_heads)

    @property
    def kv_primary(self) -> int:
        return self.rank - self.rank % self.kv_replicas

    @property
    def kv_head0(self) -> int:      # first global KV head of this rank
        return (self.rank * self.qh_l) // (self.cfg.q_heads // self.cfg.kv_heads)

    @property
    def qsa_proj_l(self) -> int:    # q+gate | k | v | indexer q+k
        c = self.cfg
        return self.qh_l * 2 * c.head_dim + 2 * self.kvh_l * c.head_dim + (c.idx_heads + 1) * c.idx_dim

    # MoE / head / PLE
    @property
    def exp_l(self) -> int:
        return self.cfg.n_experts // self.ranks

    @property
    def sffn_l(self) -> int:
        return self.cfg.ffn // self.ranks

    @property
    def vocab_l(self) -> int:
        return self.cfg.vocab // self.ranks

    @property
    def ple_kv(self) -> int:        # key rows for 4 streams + value rows
        return self.cfg.hc * self.sh + self.sh

    def cols(self) -> slice:
        """This rank's hidden columns of one stream."""
        return slice(self.rank * self.sh, (self.rank + 1) * self.sh)

    def summary(self) -> dict:
        names = ["sh", "xw", "hc_send", "gdn_vl", "gdn_kl", "gdn_qkv_l", "gdn_proj_l", "gdn_state", "qh_l",
                 "kvh_l", "kv_replicas", "qsa_proj_l", "exp_l", "sffn_l", "vocab_l", "ple_kv"]
        return {n: getattr(self, n) for n in names}
