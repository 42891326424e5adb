"""GPU <-> GPU transfer paths of this box, measured between rank r and rank r + 1 with every rank sending at once:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29534 \
        -m qwb200.tools.p2p_bench [--mb 256] [--latency-bytes 10240]

* copy-engine copy into the neighbour's memory (``cudaMemcpyAsync`` on a peer pointer of the symmetric region);
* kernel-initiated peer stores (push) and peer loads (pull) of the same bytes (the copy kernel of the host tier over
  128 segments);
* small-message latency: the time of one chained all-reduce of ``--latency-bytes`` over the peer-memory channel
  (push + flag + bounded poll: the primitive under every collective of the engine).
Device-timed, max over ranks.  The pool's reference figure for a peer copy is 770 GB/s per direction.
(The reference's bench/p2p_bench.hip and bench/uncached_bench.hip measure the same paths on PCIe.)"""
import argparse
import ctypes as C
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--latency-bytes", type=int, default=10240)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    from qwb200.ops import lib as qlib
    from qwb200.parallel.dist_engine import SymmetricRegion
    L = qlib.load(True)
    n = a.mb << 20
    reg = SymmetricRegion(n, dev)
    src = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev)
    nxt = (rank + 1) % world
    peer, mine = reg.ptrs[nxt], reg.ptrs[rank]
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    nseg = 128
    seg = n // nseg
    offs = torch.arange(nseg, dtype=torch.int64) * seg
    tab = lambda base: (offs + base).to(dev)
    by = torch.full((nseg,), seg, dtype=torch.int64, device=dev)
    t_src, t_peer, t_mine, t_dst = tab(src.data_ptr()), tab(peer), tab(mine), tab(src.data_ptr())
    P = lambda t: C.c_void_p(t.data_ptr())
    out = {"ranks": world, "mb": a.mb}

    def timed(name, fn, iters, nbytes=None):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
        out[name] = {"ms": round(ms, 4)}
        if nbytes:
            out[name]["gb_s_per_direction"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        if rank == 0:
            print(f"{name:34s} {ms * 1e3:10.1f} us" + (f"  {out[name]['gb_s_per_direction']:8.1f} GB/s per direction" if nbytes else ""), flush=True)
    timed("copy engine -> peer", lambda: L.qwk_memcpy_async(C.c_void_p(peer), P(src), C.c_longlong(n), 3, s), a.iters, n)
    timed("kernel push (peer stores)", lambda: L.qwk_segments_copy(P(t_src), P(t_peer), P(by), nseg, s), a.iters, n)
    timed("kernel pull (peer loads)", lambda: L.qwk_segments_copy(P(t_peer), P(t_dst), P(by), nseg, s), a.iters, n)
    timed("kernel copy, local", lambda: L.qwk_segments_copy(P(t_src), P(t_mine), P(by), nseg, s), a.iters, 0)
    # small-message latency through the prefill channel's stand-alone all-reduce
    from qwb200.models.config import ModelConfig, ShardConfig
    from qwb200.ops import structs as S
    from qwb200.parallel import tp_channel
    cfg = ModelConfig.full()
    sc = ShardConfig(cfg, world, rank)
    ch = tp_channel.make_symmetric(cfg, sc, 64, dev, mtp=False)
    cols = 320
    rows = max(1, a.latency_bytes // (cols * 4))
    x = torch.randn(rows, cols, device=dev)
    y = torch.zeros(rows, cols, device=dev)
    timed(f"all-reduce of {rows * cols * 4} bytes, chained", lambda: L.qwk_tp_allreduce(ch.ptr, S.TP_DOWN, P(x), P(y), rows, cols, s), 500)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
