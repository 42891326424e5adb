#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tokens/s of the full 180B hybrid MoE (random-init q4
experts, bf16 dense weights and activations) after a 4,096-token random context, on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W           # this engine
    python bench.py --impl reference ...                    # the unmodified reference (HIP-only: unavailable)

Prints one JSON line from rank 0.  ``value`` is timed on the device with CUDA events around K
chained graph replays (the sampled token is fed back on the device), max over ranks; ``e2e`` is the
same metric through ``Engine.decode`` — the public per-step call — with the step's row table copied
from pinned host memory and the sampled token read back to the host every step.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_DECODE_TOK_S = 67.0      # reference, 4x V620, plain decode batch 1


def log(msg):
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"[bench] {msg}", file=sys.stderr, flush=True)


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a HIP/ROCm engine for gfx1030 (CMake, hipcc, rocBLAS): it has no Python "
                      "package to install and cannot be built or run on a CUDA box"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--model", default="full", choices=["full", "slice2", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="debug: run a model with fewer layers (marks the result invalid)")
    ap.add_argument("--ple-rows", type=int, default=1 << 22)
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end loop (default: --steps)")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "p2p-unfused", "p2p-mute", "nccl"],
                    help="multi-GPU collectives: this library's peer-memory kernels, or the NCCL baseline")
    ap.add_argument("--fuse-kinds", type=int, default=7,
                    help="timing diagnostic (results are wrong unless 7): bit mask of the fused collective kinds that run "
                         "(1 all-reduce, 2 all-gather, 4 reduce-scatter)")
    ap.add_argument("--profile-step", action="store_true",
                    help="bracket one extra chained decode step with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.engine import device_model as DM
    from qwb200.models.config import ModelConfig
    from qwb200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        log(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(dev))

    W, K = max(3, args.warmup), args.steps
    cfg = {"full": ModelConfig.full, "slice2": ModelConfig.slice2, "tiny": ModelConfig.tiny}[args.model]()
    valid = args.model == "full" and not args.layers
    if args.layers:
        cfg = ModelConfig(**{**cfg.__dict__, "n_layers": args.layers})
    e2e_steps = args.e2e_steps or K
    need = args.context + 2 * (W + K) + 2 * (W + e2e_steps) + 64
    opts = EngineOptions(slots=1, slot_tokens=need, use_graphs=True, save_gdn=True)      # GDN state saves after every row: speculative verification
    t0 = time.time()
    if world > 1:
        from qwb200.parallel.dist_engine import make_engine
        eng = make_engine(cfg, opts, world, rank, dev, ple_rows=args.ple_rows, log=log, comm=args.comm)
        if args.fuse_kinds != 7:
            from qwb200.ops import lib as qlib
            qlib.load(True).qwrt_set_fuse_kinds(args.fuse_kinds)
    else:
        eng = Engine.synthetic(cfg, opts, device=dev, ple_rows=args.ple_rows, log=log)
    log(f"model ready in {time.time() - t0:.1f} s: {eng.dm.weight_bytes() / 1e9:.1f} GB of weights on rank {rank}")

    # ---- context: 4,096 random tokens through the prefill path (untimed)
    g = torch.Generator().manual_seed(1234)
    ctx = torch.randint(0, cfg.vocab, (args.context,), generator=g).tolist()
    token_major = bool(eng.opts.prefill_chunk) and (world == 1 or eng.tp_channels is not None)
    if token_major:
        eng.prefill(0, ctx[:512], want_logits=False)      # warm the prefill path (buffers, kernel attributes), then start over
        torch.cuda.synchronize()
        eng.reset(0)
    t0 = time.time()
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pe0.record()
    eng.prefill(0, ctx, want_logits=True)
    pe1.record()
    torch.cuda.synchronize()
    prefill_ms = pe0.elapsed_time(pe1)
    eng.dm.check_error()
    first = int(eng.dm.buf["amax_idx"][eng.last_prefill_row])
    log(f"context of {args.context} tokens in {time.time() - t0:.2f} s")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    chained = eng.merge_argmax is None      # the NCCL baseline merges the argmax on the host side of the graph

    def run_steps(tok, n):
        if chained:
            return eng.decode_chain(0, tok, n)
        out = []
        for _ in range(n):
            tok = eng.decode([0], [tok])[0]
            out.append(tok)
        return out

    # ---- device-timed: chained greedy decode, one graph replay per token
    toks = run_steps(first, W)
    launches = int(eng.dm.lib.qwrt_last_launches()) if hasattr(eng.dm.lib, "qwrt_last_launches") else 0
    if args.profile_step:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        toks = run_steps(toks[-1], 1)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    toks2 = run_steps(toks[-1], K)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    # ---- end to end: Engine.decode per token (pinned H2D of the row table, D2H of the token)
    t = toks2[-1]
    for _ in range(W):
        t = eng.decode([0], [t])[0]
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        t = eng.decode([0], [t])[0]
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    sampler.stop()
    # ---- speculative decoding (one GPU): cost of a step with 3 drafts.  Random weights accept almost nothing, so the
    # throughput the reference quotes (which rests on 2.35-3.53 accepted tokens per step with real weights) is given
    # as a derived figure at its published 2.5 tokens per step, next to what was actually measured here.
    mtp = None
    if world == 1 and eng.mtp:
        kd = 3
        eng.reset(0)
        eng.prefill(0, ctx[:512])
        tk = int(eng.dm.buf["amax_idx"][eng.last_prefill_row])
        got = eng.generate_greedy(0, tk, 8, k=kd)            # warm-up: captures the draft / verify graphs
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        got = eng.generate_greedy(0, got[-1], 48, k=kd)
        s1.record()
        torch.cuda.synchronize()
        spec_ms = s0.elapsed_time(s1)
        steps_, acc_ = max(1, eng.spec_steps), eng.spec_accepted
        # phase split (host-timed with a synchronise after each phase)
        ph = {"draft": 0.0, "verify": 0.0, "accept": 0.0}
        pend = got[-1]
        for _ in range(16):
            torch.cuda.synchronize(); a0 = time.perf_counter()
            dr = eng.draft(0, pend, kd)
            torch.cuda.synchronize(); a1 = time.perf_counter()
            lg = eng.verify(0, [pend] + dr)
            torch.cuda.synchronize(); a2 = time.perf_counter()
            pend = int(lg[0].argmax())
            a2b = time.perf_counter()
            eng.accept(0, [pend] + dr, 1)
            torch.cuda.synchronize(); a3 = time.perf_counter()
            ph["draft"] += (a1 - a0) * 1e3 / 16; ph["verify"] += (a2 - a1) * 1e3 / 16; ph["accept"] += (a3 - a2b) * 1e3 / 16
        per_step = spec_ms / steps_
        mtp = {"drafts": kd, "ms_per_spec_step": round(per_step, 3), "spec_steps": steps_, "accepted_drafts": acc_,
               "phase_ms": {k_: round(v_, 3) for k_, v_ in ph.items()},
               "tokens_per_step_measured": round(48 / steps_, 3), "tok_s_measured_random_weights": round(48 / (spec_ms / 1e3), 1),
               "tok_s_at_2.5_tokens_per_step": round(2.5 / (per_step / 1e3), 1),
               "note": "derived: measured step cost x the reference's published acceptance; random weights cannot show acceptance"}
    if dist is not None:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(tt[0]), float(tt[1])
    clocks = sampler.summary()
    if rank == 0:
        val = K / (ms / 1e3)
        out = {
            "metric": "plain decode tok/s (batch 1, greedy, 4,096-token context, CUDA-graph decode)",
            "value": round(val, 2), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(val / BASELINE_DECODE_TOK_S, 3), "dtype": "bf16 activations + q4 experts",
            "data": "synthetic (random-init weights, random token context, synthetic fp8 PLE table)",
            "config": {"model": "Qwen3.8-Flash-Next 180B hybrid MoE" if valid else f"{args.model} layers={cfg.n_layers} (not the named model)",
                       "global_batch": 1, "seq_len": args.context,
                       "parallelism": f"tp{world}+ep{world} ({args.comm} collectives)" if world > 1 else "single GPU",
                       "l2": "inputs larger than L2: every step streams ~9.8 GB of weights",
                       "ple_rows": args.ple_rows, "generated": K},
            "clocks": clocks,
            "e2e": {"value": round(e2e_steps / (ms_e2e / 1e3), 2), "unit": "tok/s", "steps": e2e_steps,
                    "h2d_bytes_per_step": int(eng.dm.rows_host.numel() * 4), "d2h_bytes_per_step": 4,
                    "api": "Engine.decode"},
            "prefill": {"tokens": args.context, "ms": round(prefill_ms, 2), "tok_s": round(args.context / (prefill_ms / 1e3), 1),
                        "path": "token-major" if token_major else "row-batched",
                        "lanes": (eng.prefiller.lanes if eng.prefiller is not None else 0)},
            "mtp": mtp,
            "gpu_launches": launches * K,
            "gpu_launches_per_step": launches,
            "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
