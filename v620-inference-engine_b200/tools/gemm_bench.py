"""Throughput of the tcgen05 GEMM on the prefill shapes against cuBLAS (torch.matmul), CUDA-event
timed with operands rotated through a set larger than L2:  python -m qwb200.tools.gemm_bench [--tokens 4096]"""
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
    a = ap.parse_args()
    T = a.tokens
    peak = 1600.0
    p = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p))["bf16_tflops"]
    for name, (N, Kd) in SHAPES.items():
        copies = max(2, int(300e6 // (N * Kd * 2 + T * Kd * 2)) + 1)
        Ws = [(torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        As = [torch.randn(T, Kd, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        i = [0]

        def ours():
            i[0] = (i[0] + 1) % copies
            K.gemm_bf16_tc(As[i[0]], Ws[i[0]], out=out)

        def cublas():
            i[0] = (i[0] + 1) % copies
            torch.matmul(As[i[0]], Ws[i[0]].T, out=out)
        t1, t2 = time_fn(ours), time_fn(cublas)
        fl = 2.0 * T * N * Kd / 1e9
        print(f"{name:14s} T={T} N={N:6d} K={Kd:5d}: tcgen05 {t1 * 1e3:8.1f} us {fl / t1:7.1f} TFLOP/s ({100 * fl / t1 / peak:4.1f}% of measured cuBLAS peak) | "
              f"cuBLAS {t2 * 1e3:8.1f} us {fl / t2:7.1f} TFLOP/s", flush=True)


if __name__ == "__main__":
    main()
