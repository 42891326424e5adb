"""Cost of one dependent kernel boundary inside a CUDA graph, with and without programmatic
dependent launch:  python -m qwb200.tools.launch_bench"""
import ctypes as C

import torch

from ..ops import lib as qlib


def main():
    lib = qlib.load(required=True)
    lib.qwk_bench_chain.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    p = torch.zeros(1024, device="cuda")
    for blocks in (1, 148, 592):
        for pdl in (0, 1):
            n = 500
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                lib.qwk_bench_chain(C.c_void_p(p.data_ptr()), 4, blocks, pdl, C.c_void_p(st.cuda_stream))
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    lib.qwk_bench_chain(C.c_void_p(p.data_ptr()), n, blocks, pdl, C.c_void_p(st.cuda_stream))
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                for _ in range(10):
                    g.replay()
                e1.record(st)
                torch.cuda.synchronize()
            print(f"blocks={blocks:4d} pdl={pdl}: {e0.elapsed_time(e1) * 1e3 / (10 * n):.2f} us per dependent kernel")


if __name__ == "__main__":
    main()
