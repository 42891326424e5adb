"""Latency of the decode-sized collectives, chained back to back, device-timed, max over ranks:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m qwb200.tools.comm_bench [--iters 2000]

Measures the stand-alone peer-memory kernels (all-reduce of the 1,300-float mixer vector = 5.2 KB, reduce-scatter of a
[rows][hidden] fp32 block output, all-gather of the bf16 block input) and the same collectives through NCCL.  The fused
forms have no launch of their own.  With ``--prefill-rows T`` it also times the prefill-sized collectives of a T-row chunk
over the prefill channel (``ops/csrc/tp.cuh``, stand-alone push + reduce kernels): the block-input all-gather (T x H bf16),
the block-output reduce-scatter (T x H fp32), the mixer all-reduce (T x 328 fp32), with the bytes each rank sends over
NVLink and the GB/s that makes, against NCCL on the same payloads.
(The reference's figure for the chained 5.2 KB all-reduce on PCIe: 45.7 -> 15.7 us, its design document under docs/, lines 238 and 1586.)"""
import argparse
import ctypes as C
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=2000)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--prefill-rows", type=int, default=0, help="also time the collectives of a prefill chunk of this many rows")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.parallel.dist_engine import attach_p2p
    cfg = ModelConfig.full()
    import dataclasses
    small = dataclasses.replace(cfg, n_layers=1, layer_types=("gdn",))          # the collectives only need the shapes
    eng = Engine.synthetic(small, EngineOptions(slots=1, slot_tokens=256, use_graphs=False), ranks=world, rank=rank, device=dev,
                           ple_rows=1 << 12)
    attach_p2p(eng)
    dm, L, sc = eng.dm, eng.dm.lib, eng.dm.sc
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p2p = dm.model.p2p
    M, ld = a.rows, sc.hc_send
    out = {}

    def timed(name, fn, nbytes):
        for _ in range(20):
            fn(0)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = {"us": round(float(t), 2), "bytes": nbytes}
        if rank == 0:
            print(f"{name:28s} {float(t):8.2f} us per collective ({nbytes} bytes per rank)", flush=True)

    k = [0]

    def bump():
        k[0] += 1
        if k[0] % 4000 == 0:
            L.qwk_p2p_bump_base(p2p, 4096, s)
        return (k[0] % 4000) + 1
    send, red, part, outb = dm.buf["send"], dm.buf["red"], dm.buf["partial"], dm.buf["out_a"]
    timed("p2p all-reduce 5.2 KB", lambda i: L.qwk_p2p_allreduce(p2p, bump(), C.c_void_p(send.data_ptr()), C.c_void_p(red.data_ptr()), M, ld, s), M * ld * 4)
    timed("p2p reduce-scatter [rows][H]", lambda i: L.qwk_p2p_reduce_scatter(p2p, bump(), C.c_void_p(part.data_ptr()), C.c_void_p(outb.data_ptr()), M, sc.sh, s), M * cfg.hidden * 4)
    timed("p2p all-gather bf16 [rows][H]", lambda i: L.qwk_p2p_allgather(p2p, bump(), 1, dm.model.off_bin, M, sc.sh, 2, s), M * sc.sh * 2)
    x = torch.zeros(M * ld, device=dev)
    timed("nccl all-reduce 5.2 KB", lambda i: dist.all_reduce(x), M * ld * 4)
    y, yo = torch.zeros(world, M * sc.sh, device=dev), torch.zeros(M * sc.sh, device=dev)
    timed("nccl reduce-scatter [rows][H]", lambda i: dist.reduce_scatter_tensor(yo, y), M * cfg.hidden * 4)
    if a.prefill_rows:
        from qwb200.ops import structs as S
        from qwb200.parallel import tp_channel
        T = a.prefill_rows
        ch = tp_channel.make_symmetric(cfg, sc, T, torch.device(dev), mtp=False)
        a.iters = max(20, a.iters // 20)
        H, SH = cfg.hidden, sc.sh
        bin_slice = torch.randn(T, SH, device=dev).to(torch.bfloat16)
        block_out = torch.randn(T, H, device=dev)
        rs_out = torch.zeros(T, SH, device=dev)
        dn = torch.randn(T, 328, device=dev)
        dn_out = torch.zeros(T, 328, device=dev)
        P = lambda t: C.c_void_p(t.data_ptr())
        sent = lambda total: total * (world - 1) // world          # bytes this rank puts on the links
        timed(f"tp all-gather {T}xH bf16", lambda i: L.qwk_tp_allgather(ch.ptr, S.TP_BIN, P(bin_slice), SH * 2, T, SH * 2, 1, s), T * SH * 2 * (world - 1))
        timed(f"tp reduce-scatter {T}xH fp32", lambda i: L.qwk_tp_reduce_scatter(ch.ptr, S.TP_RS, P(block_out), P(rs_out), T, SH, s), sent(T * H * 4))
        timed(f"tp all-reduce {T}x328 fp32", lambda i: L.qwk_tp_allreduce(ch.ptr, S.TP_DOWN, P(dn), P(dn_out), T, 328, s), T * 328 * 4 * (world - 1))
        g_in, g_out = bin_slice, torch.zeros(world, T, SH, dtype=torch.bfloat16, device=dev)
        timed(f"nccl all-gather {T}xH bf16", lambda i: dist.all_gather_into_tensor(g_out, g_in), T * SH * 2 * (world - 1))
        r_in = block_out.view(T, world, SH).permute(1, 0, 2).contiguous()
        timed(f"nccl reduce-scatter {T}xH fp32", lambda i: dist.reduce_scatter_tensor(rs_out, r_in), sent(T * H * 4))
        timed(f"nccl all-reduce {T}x328 fp32", lambda i: dist.all_reduce(dn_out), T * 328 * 4 * (world - 1))
        for k_, v in out.items():
            if k_.startswith(("tp ", "nccl ")) and str(T) in k_:
                v["gb_s_sent_per_rank"] = round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1)
                if rank == 0:
                    print(f"{k_:34s} {v['gb_s_sent_per_rank']:8.1f} GB/s sent per rank", flush=True)
    dm.check_error()
    if rank == 0:
        print(json.dumps({"ranks": world, "rows": M, **out}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
