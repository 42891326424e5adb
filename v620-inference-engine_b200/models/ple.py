"""Host-resident n-gram PLE table ("sidecar").

On disk: ``META.json {layout, width, rows, shards, scale}`` plus ``shard_<i>.safetensors``;
row ``r`` lives in shard ``r // rows_per_shard``.  Four layouts (reference src/core/ple.cpp:127-211):

* ``group16_int4_fp16scale_lownibblefirst`` – ``weight_i4`` u8 ``[rows, width/2]`` + ``weight_scale`` f16 ``[rows, width/16]``
* ``group16_int8_fp16scale``                – ``weight_i8`` i8 ``[rows, width]`` + ``weight_scale`` f16
* ``bf16``                                  – ``weight`` bf16 ``[rows, width]``
* ``f8e4m3_tensorscale``                    – ``weight_f8`` u8 ``[rows, width]`` with one tensor scale (256-entry LUT)

In memory the table is one pinned host tensor per shard (or one for all shards), so the GPU
gather kernel can read rows straight out of host RAM; ``gather`` is the CPU path used by the
oracle and the tests.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional

import numpy as np
import torch

from .config import ModelConfig
from .ngram import NgramHasher

LAYOUTS = {
    "group16_int4_fp16scale_lownibblefirst": "int4",
    "group16_int8_fp16scale": "int8",
    "bf16": "bf16",
    "f8e4m3_tensorscale": "f8",
}


def f8e4m3_lut(scale: float = 1.0) -> torch.Tensor:
    """fp32 value of each of the 256 E4M3 (finite-only "fn" variant) bit patterns times ``scale``."""
    b = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    v = b.view(torch.float8_e4m3fn).float()
    v = torch.nan_to_num(v, nan=0.0)
    return v * scale


class PleTable:
    def __init__(self, cfg: ModelConfig, layout: str, shards: List[dict], rows: int, rows_per_shard: int,
                 scale: float = 1.0):
        assert layout in LAYOUTS.values()
        self.cfg, self.layout, self.shards, self.rows = cfg, layout, shards, rows
        self.rows_per_shard, self.scale = rows_per_shard, scale
        self.width = cfg.ngram_dim
        self.lut = f8e4m3_lut(scale) if layout == "f8" else None

    # ---- construction
    @staticmethod
    def synthetic(cfg: ModelConfig, rows: Optional[int] = None, layout: str = "f8", n_shards: int = 1, seed: int = 0,
                  pin: bool = False, scale: float = 0.25) -> "PleTable":
        """Random table: values N(0,1) (clipped to the format's range) times ``scale``.  ``rows``
        defaults to the hasher's vocabulary; pass a smaller count to scale the table down — ids
        are then reduced modulo ``rows`` by the caller (``PleTable.wrap``)."""
        hasher = NgramHasher(cfg)
        rows = rows or hasher.total_rows
        rps = (rows + n_shards - 1) // n_shards
        g = torch.Generator().manual_seed(seed)
        w = cfg.ngram_dim
        shards = []
        for s in range(n_shards):
            n = min(rps, rows - s * rps)
            if layout == "f8":
                # byte-level synthesis: uniform random E4M3 patterns would be far from normal, so
                # draw normals in blocks and convert
                t = torch.empty((n, w), dtype=torch.uint8)
                step = 1 << 20
                for a in range(0, n, step):
                    m = min(step, n - a)
                    x = torch.randn((m, w), generator=g).clamp_(-448, 448)
                    t[a:a + m] = x.to(torch.float8_e4m3fn).view(torch.uint8)
                sh = {"weight_f8": t}
            elif layout == "bf16":
                sh = {"weight": (torch.randn((n, w), generator=g) * scale).to(torch.bfloat16)}
            elif layout == "int8":
                x = torch.randn((n, w), generator=g) * scale
                xs = x.reshape(n, w // 16, 16)
                sc = (xs.abs().amax(-1) / 127).clamp_min(1e-8).to(torch.float16)
                q = torch.round(xs / sc.float().unsqueeze(-1)).clamp_(-127, 127).to(torch.int8).reshape(n, w)
                sh = {"weight_i8": q, "weight_scale": sc}
            else:
                x = torch.randn((n, w), generator=g) * scale
                xs = x.reshape(n, w // 16, 16)
                sc = (xs.abs().amax(-1) / 7).clamp_min(1e-8).to(torch.float16)
                q = (torch.round(xs / sc.float().unsqueeze(-1)).clamp_(-8, 7) + 8).to(torch.uint8).reshape(n, w // 2, 2)
                sh = {"weight_i4": (q[..., 0] | (q[..., 1] << 4)).contiguous(), "weight_scale": sc}
            if pin and torch.cuda.is_available():
                sh = {k: v.pin_memory() for k, v in sh.items()}
            shards.append(sh)
        return PleTable(cfg, layout, shards, rows, rps, scale if layout == "f8" else 1.0)

    def save(self, d: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(d, exist_ok=True)
        name = {v: k for k, v in LAYOUTS.items()}[self.layout]
        with open(os.path.join(d, "META.json"), "w") as f:
            json.dump({"layout": name, "width": self.width, "rows": self.rows, "shards": len(self.shards),
                       "scale": self.scale}, f)
        for i, sh in enumerate(self.shards):
            save_file({k: v.contiguous() for k, v in sh.items()}, os.path.join(d, f"shard_{i}.safetensors"))

    @staticmethod
    def load(cfg: ModelConfig, d: str, pin: bool = False) -> "PleTable":
        from safetensors.torch import load_file
        with open(os.path.join(d, "META.json")) as f:
            meta = json.load(f)
        if meta["layout"] not in LAYOUTS:
            raise ValueError(f"PLE sidecar: unsupported layout {meta['layout']}")
        if int(meta["width"]) != cfg.ngram_dim:
            raise ValueError("PLE sidecar: width")
        rows, n = int(meta["rows"]), int(meta["shards"])
        rps = (rows + n - 1) // n
        shards = []
        for i in range(n):
            sh = load_file(os.path.join(d, f"shard_{i}.safetensors"))
            if pin and torch.cuda.is_available():
                sh = {k: v.pin_memory() for k, v in sh.items()}
            shards.append(sh)
        return PleTable(cfg, LAYOUTS[meta["layout"]], shards, rows, rps, float(meta.get("scale", 1.0)))

    # ---- access
    def wrap(self, ids: np.ndarray) -> np.ndarray:
        """Reduce hashed ids into a scaled-down table."""
        return ids % self.rows

    def rows_f32(self, ids: torch.Tensor) -> torch.Tensor:
        """ids int64 [...]  ->  fp32 [..., width]."""
        flat = ids.reshape(-1)
        out = torch.empty((flat.numel(), self.width), dtype=torch.float32)
        sid = flat // self.rows_per_shard
        rid = flat % self.rows_per_shard
        for s in range(len(self.shards)):
            m = sid == s
            if not bool(m.any()):
                continue
            r = rid[m]
            sh = self.shards[s]
            if self.layout == "f8":
                out[m] = self.lut[sh["weight_f8"][r].long()]
            elif self.layout == "bf16":
                out[m] = sh["weight"][r].float()
            elif self.layout == "int8":
                q = sh["weight_i8"][r].float().reshape(-1, self.width // 16, 16)
                out[m] = (q * sh["weight_scale"][r].float().unsqueeze(-1)).reshape(-1, self.width)
            else:
                b = sh["weight_i4"][r].to(torch.int32)
                q = torch.stack([(b & 0xF) - 8, (b >> 4) - 8], dim=-1).float().reshape(-1, self.width // 16, 16)
                out[m] = (q * sh["weight_scale"][r].float().unsqueeze(-1)).reshape(-1, self.width)
        return out.reshape(*ids.shape, self.width)

    def gather(self, ids) -> torch.Tensor:
        """ids [T, heads] -> e [T, heads*width] fp32 (the concatenation of the heads' rows)."""
        ids = torch.as_tensor(np.asarray(ids), dtype=torch.int64)
        ids = ids % self.rows
        T = ids.shape[0]
        return self.rows_f32(ids).reshape(T, -1)

    @property
    def nbytes(self) -> int:
        return sum(v.numel() * v.element_size() for sh in self.shards for v in sh.values())
