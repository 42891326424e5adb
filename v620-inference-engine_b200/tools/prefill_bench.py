"""Prefill throughput and where the time goes, on one GPU or on N (one process per GPU under torchrun):

    python -m qwb200.tools.prefill_bench [--tokens 4096] [--chunk 4096] [--ctx 0] [--layers 0] [--lanes 0] [--by-step]
                                         [--tokens-file ids.txt] [--energy]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m qwb200.tools.prefill_bench ...

Tokens per second of one prompt through the token-major path (CUDA events on the launching stream, max over ranks), then,
with ``--by-step``, a second pass in which the native runtime brackets every step of a chunk with events and adds the
device time up per category (mixer glue / mixer GEMMs / projections / GDN / QSA / out projection (+ reduce-scatter) /
routing / expert GEMMs / shared down + combine / PLE / MTP pass / guard waits).  On several ranks a step's time
includes what it waits for inside the kernel, which is the point.  ``--tokens-file`` takes the prompt (context first, then
the measured part) from a file of token ids instead of random ids: real text routes to fewer distinct experts per chunk
and re-selects attention groups, so its numbers differ from the random-token floor.  ``--energy`` integrates this rank's
GPU power (NVML) over the best timed repetition and reports joules per prompt token.

(The reference's tool: bench/prefill_bench with --ctx / --tokens-file.)"""
import argparse
import ctypes as C
import dataclasses
import json
import os

import torch

from ..engine.engine import Engine, EngineOptions
from ..models.config import ModelConfig

def read_token_file(path: str, vocab: int):
    """Token ids separated by white space and / or commas; ids outside the vocabulary are refused."""
    with open(path) as f:
        ids = [int(x) for x in f.read().replace(",", " ").split()]
    bad = [t for t in ids if not 0 <= t < vocab]
    if bad:
        raise ValueError(f"{path}: {len(bad)} ids outside the vocabulary (first: {bad[0]})")
    return ids


CATS = ["mixer pre-norm (+ pending block output)", "mixer GEMMs", "projection GEMM", "GDN conv + scan", "QSA prep / scores / select / attend", "out projection",
        "router GEMM + routing + sort", "expert GEMMs + swiglu", "shared down + combine", "PLE", "other", "MTP pass", "guard waits", "mixer norm (after the sums of squares)", "mixer mid (after the down projection)",
        "mixer mix (+ block-input all-gather)"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--ctx", type=int, default=0, help="tokens already in the slot before the measured prompt")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--lanes", type=int, default=0, help="micro-batches per chunk (0: the default of the rank count)")
    ap.add_argument("--by-step", action="store_true", help="a second pass with the runtime's per-category step timing")
    ap.add_argument("--repeat", type=int, default=2, help="timed repetitions (the best is reported)")
    ap.add_argument("--tokens-file", default=None, help="token ids of the prompt (context + measured part) instead of random ids")
    ap.add_argument("--energy", action="store_true", help="integrate this rank's GPU power over each timed repetition")
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg = ModelConfig.full()
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    if a.lanes:
        from ..utils import settings
        settings.set_current(settings.Settings.from_env(prefill_lanes=a.lanes))
    opts = EngineOptions(slots=1, slot_tokens=a.ctx + a.tokens + 512, use_graphs=False, prefill_chunk=a.chunk)
    if world > 1:
        from ..parallel.dist_engine import make_engine
        eng = make_engine(cfg, opts, world, rank, dev, ple_rows=1 << 20)
    else:
        eng = Engine.synthetic(cfg, opts, device=dev, ple_rows=1 << 20)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab, (a.ctx + a.tokens,), generator=g).tolist()
    if a.tokens_file:
        toks = read_token_file(a.tokens_file, cfg.vocab)
        if len(toks) < a.ctx + a.tokens:
            raise SystemExit(f"--tokens-file holds {len(toks)} ids, --ctx + --tokens asks for {a.ctx + a.tokens}")
        toks = toks[:a.ctx + a.tokens]

    def sync():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def fresh():
        eng.reset(0)
        if a.ctx:
            eng.prefill(0, toks[:a.ctx], want_logits=False)
        sync()

    eng.prefill(0, toks[:min(512, a.tokens)], want_logits=False)          # warm-up
    best, energy = None, None
    for _ in range(max(1, a.repeat)):
        fresh()
        meter = None
        if a.energy:
            from ..utils.power import PowerMeter
            meter = PowerMeter(indices=[local]).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill(0, toks[a.ctx:], want_logits=True)
        e1.record()
        sync()
        used = meter.stop() if meter is not None else None
        eng.dm.check_error()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if best is None or float(t) < best:
            best, energy = float(t), used
    pf = eng.prefiller
    out = {"tokens": a.tokens, "ctx": a.ctx, "ranks": world, "lanes": pf.lanes, "chunk": pf.T, "ms": round(best, 2),
           "tok_s": round(a.tokens / best * 1e3), "launches_per_chunk": int(eng.dm.lib.qwrt_prefill_last_launches())}
    if energy is not None and energy.get("ok"):
        out["energy"] = {"gpu": local, "avg_w": energy["avg_w"], "joules": round(energy["kilojoules"] * 1e3, 1),
                         "joules_per_token": round(energy["kilojoules"] * 1e3 / a.tokens, 4)}
    if a.tokens_file:
        out["tokens_file"] = os.path.basename(a.tokens_file)
    if a.by_step:
        lib = eng.dm.lib
        lib.qwrt_prefill_profile.argtypes = [C.c_int]
        lib.qwrt_prefill_profile_read.argtypes = [C.POINTER(C.c_double), C.c_int]
        fresh()
        lib.qwrt_prefill_profile(1)
        eng.prefill(0, toks[a.ctx:], want_logits=True)
        lib.qwrt_prefill_profile(0)
        sync()
        buf = (C.c_double * 16)()
        n = lib.qwrt_prefill_profile_read(buf, 16)
        split = {CATS[i]: round(buf[i], 2) for i in range(min(n, len(CATS)))}
        out["split_ms"] = split
        if rank == 0:
            tot = sum(split.values()) or 1.0
            for k, v in sorted(split.items(), key=lambda kv: -kv[1]):
                print(f"  {k:40s} {v:8.2f} ms  {100 * v / tot:5.1f} %", flush=True)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
