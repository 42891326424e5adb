"""Bandwidth of the decode matrix-vector kernels on the model's shapes, timed inside a CUDA graph
with a rotating set of weight matrices larger than L2 (so every launch streams from HBM):

    python -m qwb200.tools.gemv_bench [--rows 1 2 8 16]

Reports microseconds per launch and achieved TB/s against the measured copy bandwidth
(role of the reference's bench/gemm_bench.hip for the decode shapes)."""
import argparse
import json
import os

import torch

from ..ops import kernels as K

SHAPES = {
    "gdn_proj": (16444, 2560), "qsa_proj": (13952, 2560), "out_proj": (2560, 6144), "router_shared": (1793, 2560),
    "ple_kv": (12800, 2560), "lm_head": (248320, 2560),
    "tp8_gdn_proj": (2060, 2560), "tp8_out_proj": (2560, 768), "tp8_lm_head": (31040, 2560),
}


def bench(name, N, Kd, M, reps=20, dev="cuda"):
    nbytes = N * Kd * 2
    copies = max(2, min(16, int(400e6 // nbytes) + 1))
    Ws = [(torch.randn(N, Kd, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
    out = torch.empty(M, N, device=dev)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for W in Ws:
            K.gemv_bf16(W, x, out=out)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(reps):
                for W in Ws:
                    K.gemv_bf16(W, x, out=out)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        g.replay()
        e1.record(st)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
    ref = (x.float() @ Ws[-1].float().T)
    err = float((out - ref).abs().max() / ref.abs().max())
    return us, nbytes / us / 1e6, err


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="*", default=[1, 8])
    ap.add_argument("--shapes", nargs="*", default=list(SHAPES))
    a = ap.parse_args()
    peak = 6.5
    p = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p))["hbm_gbs"] / 1e3
    for name in a.shapes:
        N, Kd = SHAPES[name]
        for M in a.rows:
            us, tbs, err = bench(name, N, Kd, M)
            print(f"{name:14s} N={N:6d} K={Kd:5d} M={M:2d}: {us:8.2f} us  {tbs:5.2f} TB/s  {100 * tbs / peak:5.1f}% of measured copy  relerr {err:.1e}", flush=True)


if __name__ == "__main__":
    main()
