"""Converts an n-gram PLE table between its on-disk forms.

Source: either a directory of raw shards ``shard_<i>.bf16`` (flat bf16 ``[rows_per_shard, width]``, what a download of
the published table leaves behind) or an existing sidecar directory (``META.json`` + ``shard_<i>.safetensors``) in any
of the four layouts.  Target: a sidecar in the chosen layout - ``bf16``, ``int8`` / ``int4`` (one fp16 scale per 16
values: max|x| / 127 or / 7) or ``f8`` (E4M3 with one tensor scale, the layout the GPU gather kernel reads at 160 bytes
per row).  Shards are converted one at a time in row blocks, so a 320M-row table never has to fit in memory, finished
shards are skipped on a re-run, and ``--worker i/n`` splits the shards over processes.  Prints the worst relative
error of every shard.  (Role of the reference's tools/ple_convert.py:1-67; fetching the raw table is out of reach
here - no network - so there is no downloader beside it.)

  python -m qwb200.tools.ple_convert --src /data/ple_raw --dst /data/ple_f8 --layout f8 --width 160
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, Iterator, Tuple

import numpy as np
import torch

from ..models.ple import LAYOUTS, f8e4m3_lut

SHORT = {v: k for k, v in LAYOUTS.items()}      # short name -> META.json name
BLOCK = 1 << 20


def encode_rows(x: torch.Tensor, layout: str, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """fp32 rows ``[n, width]`` -> the tensors of one shard in ``layout`` (short name)."""
    n, w = x.shape
    if layout == "bf16":
        return {"weight": x.to(torch.bfloat16)}
    if layout == "f8":
        return {"weight_f8": (x / scale).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)}
    xs = x.reshape(n, w // 16, 16)
    top = 127 if layout == "int8" else 7
    sc = (xs.abs().amax(-1) / top).to(torch.float16)
    sf = sc.float().unsqueeze(-1)
    q = torch.round(torch.where(sf > 0, xs / sf, torch.zeros_like(xs)))
    if layout == "int8":
        return {"weight_i8": q.clamp_(-127, 127).to(torch.int8).reshape(n, w), "weight_scale": sc}
    if layout == "int4":
        b = (q.clamp_(-8, 7) + 8).to(torch.uint8).reshape(n, w // 2, 2)
        return {"weight_i4": (b[..., 0] | (b[..., 1] << 4)).contiguous(), "weight_scale": sc}
    raise ValueError(f"unknown layout {layout!r}")


def decode_rows(sh: Dict[str, torch.Tensor], layout: str, scale: float = 1.0) -> torch.Tensor:
    """The inverse of :func:`encode_rows`: fp32 rows of one shard (or of a row slice of it)."""
    if layout == "bf16":
        return sh["weight"].float()
    if layout == "f8":
        return f8e4m3_lut(scale)[sh["weight_f8"].long()]
    if layout == "int8":
        q = sh["weight_i8"].float()
        n, w = q.shape
        return (q.reshape(n, w // 16, 16) * sh["weight_scale"].float().unsqueeze(-1)).reshape(n, w)
    b = sh["weight_i4"].to(torch.int32)
    n, w = b.shape[0], b.shape[1] * 2
    q = torch.stack([(b & 0xF) - 8, (b >> 4) - 8], dim=-1).float().reshape(n, w // 16, 16)
    return (q * sh["weight_scale"].float().unsqueeze(-1)).reshape(n, w)


class Source:
    """Row blocks of the source table, shard by shard."""

    def __init__(self, d: str, width: int):
        self.d, self.width = d, width
        meta_path = os.path.join(d, "META.json")
        if os.path.exists(meta_path):
            with open(meta_path) as f:
                m = json.load(f)
            self.raw, self.layout = False, LAYOUTS[m["layout"]]
            self.n_shards, self.rows, self.scale = int(m["shards"]), int(m["rows"]), float(m.get("scale", 1.0))
            if int(m["width"]) != width:
                raise ValueError(f"source width {m['width']} != {width}")
        else:
            names = sorted(f for f in os.listdir(d) if f.startswith("shard_") and f.endswith(".bf16"))
            if not names:
                raise FileNotFoundError(f"{d}: neither META.json nor shard_<i>.bf16")
            self.raw, self.layout, self.n_shards, self.scale = True, "bf16", len(names), 1.0
            self.rows = sum(os.path.getsize(os.path.join(d, f"shard_{i}.bf16")) for i in range(self.n_shards)) // (2 * width)

    def blocks(self, shard: int) -> Iterator[torch.Tensor]:
        if self.raw:
            mm = np.memmap(os.path.join(self.d, f"shard_{shard}.bf16"), dtype=np.uint16, mode="r")
            if mm.size % self.width:
                raise ValueError(f"shard {shard}: size is not a multiple of the row width")
            rows = mm.reshape(-1, self.width)
            for a in range(0, rows.shape[0], BLOCK):
                yield torch.from_numpy(np.ascontiguousarray(rows[a:a + BLOCK]).view(np.int16)).view(torch.bfloat16).float()
            return
        from safetensors.torch import load_file
        sh = load_file(os.path.join(self.d, f"shard_{shard}.safetensors"))
        n = next(iter(sh.values())).shape[0]
        for a in range(0, n, BLOCK):
            yield decode_rows({k: v[a:a + BLOCK] for k, v in sh.items()}, self.layout, self.scale)


def convert(src: str, dst: str, layout: str, width: int, scale: float = 0.0, worker: Tuple[int, int] = (0, 1)) -> float:
    """Returns the worst relative error (max |decoded - x| / max |x|) over the shards converted by this worker.
    ``scale`` 0 for f8 means: max|x| of shard 0 divided by 448."""
    from safetensors.torch import save_file
    s = Source(src, width)
    os.makedirs(dst, exist_ok=True)
    if layout == "f8" and scale <= 0:
        amax = max(float(b.abs().max()) for b in s.blocks(0))
        scale = max(amax, 1e-30) / 448.0
    if layout != "f8":
        scale = 1.0
    if worker[0] == 0:
        with open(os.path.join(dst, "META.json"), "w") as f:
            json.dump({"layout": SHORT[layout], "width": width, "rows": s.rows, "shards": s.n_shards, "scale": scale}, f)
    worst = 0.0
    for i in range(worker[0], s.n_shards, worker[1]):
        out = os.path.join(dst, f"shard_{i}.safetensors")
        if os.path.exists(out):
            continue
        parts, err, amax = [], 0.0, 0.0
        for x in s.blocks(i):
            enc = encode_rows(x, layout, scale)
            err = max(err, float((decode_rows(enc, layout, scale) - x).abs().max()))
            amax = max(amax, float(x.abs().max()))
            parts.append(enc)
        sh = {k: torch.cat([p[k] for p in parts]) for k in parts[0]}
        save_file(sh, out + ".tmp")
        os.replace(out + ".tmp", out)
        rel = err / max(amax, 1e-30)
        worst = max(worst, rel)
        print(f"shard {i}: {next(iter(sh.values())).shape[0]} rows, worst relative error {rel:.4f}", flush=True)
    return worst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--layout", required=True, choices=sorted(SHORT))
    ap.add_argument("--width", type=int, default=160)
    ap.add_argument("--scale", type=float, default=0.0, help="f8 tensor scale (0: from shard 0)")
    ap.add_argument("--worker", default="0/1", help="i/n: convert the shards with index % n == i")
    a = ap.parse_args(argv)
    i, n = (int(v) for v in a.worker.split("/"))
    convert(a.src, a.dst, a.layout, a.width, a.scale, (i, n))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
