"""Offline GPTQ of bf16 matrices into the q4 g128 format the expert kernels read.

Input: one or more safetensors files with bf16 / fp16 / fp32 matrices ``[out, in]`` and the Hessian file written by
``engine.calibrate.Calibrator.dump`` (``layers.<l>.<kind>.hessian``).  Every tensor whose name matches ``--pattern``
(group 1 = layer number) and whose input width equals the Hessian's is quantised with
``models.quant.quantize_q4_gptq`` and written as ``<name>_packed`` (int32, checkpoint nibble order) and ``<name>_scale``;
the round-to-nearest and GPTQ output errors (relative, under the Hessian's metric) are printed per tensor.
(Role of the reference's tools/gptq_int8.py:1-140, which produced int8 g32 sidecars for its rejected int8 decode path.)

  python -m qwb200.tools.gptq_q4 --weights mtp.safetensors --hessians /tmp/hess/hessians.safetensors \
      --pattern 'layers\\.(\\d+)\\.mlp\\.experts\\.\\d+\\.(gate|up)_proj\\.weight' --kind moe --out /tmp/q4
"""
from __future__ import annotations

import argparse
import os
import re

import torch

from ..models import quant


def hessian_error(w: torch.Tensor, wq: torch.Tensor, h: torch.Tensor) -> float:
    """tr((W - Wq) H (W - Wq)^T) / tr(W H W^T): the relative squared output error over the calibration rows."""
    d = (w - wq).double()
    hd = h.double()
    num = torch.einsum("ok,kj,oj->", d, hd, d)
    den = torch.einsum("ok,kj,oj->", w.double(), hd, w.double())
    return float(num / den.clamp_min(1e-30))


def quantise_file(path: str, hess: dict, pattern: re.Pattern, kind: str, out_dir: str, damp: float, device: str) -> int:
    from safetensors import safe_open
    from safetensors.torch import save_file
    out = {}
    with safe_open(path, framework="pt") as f:
        for name in f.keys():
            m = pattern.fullmatch(name)
            if not m:
                continue
            key = f"layers.{int(m.group(1))}.{kind}.hessian"
            if key not in hess:
                print(f"{name}: no Hessian {key}, skipped")
                continue
            w = f.get_tensor(name).float().to(device)
            h = hess[key].float().to(device)
            if w.dim() != 2 or w.shape[1] != h.shape[0] or w.shape[1] % quant.QGROUP:
                print(f"{name}: shape {tuple(w.shape)} does not fit Hessian {tuple(h.shape)}, skipped")
                continue
            p0, s0 = quant.quantize_q4(w)
            p1, s1 = quant.quantize_q4_gptq(w, h, damp=damp)
            e0 = hessian_error(w, quant.dequantize_q4(p0, s0), h)
            e1 = hessian_error(w, quant.dequantize_q4(p1, s1), h)
            print(f"{name}: rtn {e0:.3e}  gptq {e1:.3e}")
            out[name + "_packed"] = p1.cpu()
            out[name + "_scale"] = s1.cpu()
    if out:
        os.makedirs(out_dir, exist_ok=True)
        save_file(out, os.path.join(out_dir, os.path.basename(path)))
    return len(out) // 2


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--weights", nargs="+", required=True)
    ap.add_argument("--hessians", required=True)
    ap.add_argument("--pattern", required=True, help="regex over tensor names; group 1 is the layer number")
    ap.add_argument("--kind", default="moe", choices=["attn", "moe"], help="which block input's Hessian to use")
    ap.add_argument("--out", required=True)
    ap.add_argument("--damp", type=float, default=0.01)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from safetensors.torch import load_file
    hess = load_file(a.hessians)
    pat = re.compile(a.pattern)
    n = sum(quantise_file(p, hess, pat, a.kind, a.out, a.damp, a.device) for p in a.weights)
    print(f"{n} tensors written to {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
