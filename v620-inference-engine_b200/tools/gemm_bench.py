"""Throughput of the tcgen05 GEMM on the prefill shapes against cuBLAS (torch.matmul), CUDA-event
timed with operands rotated through a set larger than L2:

    python -m qwb200.tools.gemm_bench [--tokens 4096] [--fp32] [--wide MIN_N] [--pair MIN_N] [--stage-local]

``--wide`` / ``--pair`` set from which width on the 128 x 256 tile form / the CTA-pair form (256 x 256 tiles,
tcgen05.mma.cta_group::2) is used (0 = never); ``--stage-local`` writes fp32 output through the epilogue's staging
buffers; ``--fp32`` measures fp32 output instead of bf16."""
import argparse
import json
import os

import torch

from ..ops import kernels as K

SHAPES = {"gdn_proj": (16444, 2560), "qsa_proj": (13952, 2560), "out_proj": (2560, 6144), "hc_down": (324, 10240),
          "hc_up": (10240, 320), "router": (512, 2560), "lm_head_shard": (31040, 2560)}


def time_fn(fn, reps=10):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--wide", type=int, default=-1)
    ap.add_argument("--pair", type=int, default=-1)
    ap.add_argument("--stage-local", action="store_true")
    a = ap.parse_args()
    from ..ops import lib as qlib
    L = qlib.load(True)
    if a.wide >= 0:
        L.qwk_gemm_tc_wide_min_n(a.wide)
    if a.pair >= 0:
        L.qwk_gemm_tc_pair_min_n(a.pair)
    if a.stage_local:
        L.qwk_gemm_tc_stage_local(1)
    T = a.tokens
    peak = 1600.0
    p = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p))["bf16_tflops"]
    for name, (N, Kd) in SHAPES.items():
        copies = max(2, int(300e6 // (N * Kd * 2 + T * Kd * 2)) + 1)
        Ws = [(torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        As = [torch.randn(T, Kd, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        out = torch.empty(T, N, dtype=torch.float32 if a.fp32 else torch.bfloat16, device="cuda")
        i = [0]

        def ours():
            i[0] = (i[0] + 1) % copies
            K.gemm_bf16_tc(As[i[0]], Ws[i[0]], out=out)

        def cublas():
            i[0] = (i[0] + 1) % copies
            if a.fp32:
                torch.matmul(As[i[0]], Ws[i[0]].T)          # cuBLAS bf16 output (torch has no bf16 x bf16 -> fp32 matmul): its best case
            else:
                torch.matmul(As[i[0]], Ws[i[0]].T, out=out)
        t1, t2 = time_fn(ours), time_fn(cublas)
        fl = 2.0 * T * N * Kd / 1e9
        print(f"{name:14s} T={T} N={N:6d} K={Kd:5d}: tcgen05 {t1 * 1e3:8.1f} us {fl / t1:7.1f} TFLOP/s ({100 * fl / t1 / peak:4.1f}% of measured cuBLAS peak) | "
              f"cuBLAS {t2 * 1e3:8.1f} us {fl / t2:7.1f} TFLOP/s", flush=True)


if __name__ == "__main__":
    main()
