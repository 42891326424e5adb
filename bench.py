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
    ap.add_argument("--comm", default="p2p", choices=["p2p", "p2p-unfused", "nccl"],
                    help="multi-GPU collectives: this library's peer-memory kernels (inside the compute kernels, or as kernels "
                         "of their own), or the NCCL baseline")
    ap.add_argument("--prefill-long", type=int, default=32768, help="tokens of the long-prompt prefill run (4,096-token chunks); 0 = skip")
    ap.add_argument("--mtp-context", type=int, default=8192, help="context of the speculative-decoding runs; 0 = skip them")
    ap.add_argument("--mtp-steps", type=int, default=12, help="timed speculative steps per forced-acceptance value")
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
        # in the product arm NCCL serves rendezvous and timing only: its in-switch (NVLS) transport is left off unless asked for
        # (NCCL_NVLS_ENABLE=1, e.g. for the --comm nccl baseline), so that a rank that dies does not leave its memory bound to a
        # multicast object the other ranks still use
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device(dev))

    W, K = max(3, args.warmup), args.steps
    cfg = {"full": ModelConfig.full, "slice2": ModelConfig.slice2, "tiny": ModelConfig.tiny}[args.model]()
    valid = args.model == "full" and not args.layers
    if args.layers:
        cfg = ModelConfig(**{**cfg.__dict__, "n_layers": args.layers})
    e2e_steps = args.e2e_steps or K
    need = max(args.context + 2 * (W + K) + 2 * (W + e2e_steps) + 64, args.prefill_long + 256, args.mtp_context + 1024)
    # four slots (the concurrent-stream runs); GDN state saved after every row of a step: speculative verification
    opts = EngineOptions(slots=4, slot_tokens=need, use_graphs=True, save_gdn=True)
    t0 = time.time()
    if world > 1:
        from qwb200.parallel.dist_engine import make_engine
        eng = make_engine(cfg, opts, world, rank, dev, ple_rows=args.ple_rows, log=log, comm=args.comm)
    else:
        eng = Engine.synthetic(cfg, opts, device=dev, ple_rows=args.ple_rows, log=log)
    log(f"model ready in {time.time() - t0:.1f} s: {eng.dm.weight_bytes() / 1e9:.1f} GB of weights on rank {rank}")

    # ---- context: 4,096 random tokens through the prefill path (untimed)
    g = torch.Generator().manual_seed(1234)
    ctx = torch.randint(0, cfg.vocab, (args.context,), generator=g).tolist()
    token_major = bool(eng.opts.prefill_chunk) and (world == 1 or eng.tp_channels is not None)
    t0 = time.time()
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prefill_note = None
    # under a lock-step guard: a failure that shows on some ranks only makes every rank fall back together
    from qwb200.utils.lockstep import Lockstep
    first_try = Lockstep(dist, dev, check=eng.dm.check_error, sync=torch.cuda.synchronize)

    def fill_context():
        if token_major:
            eng.prefill(0, ctx[:512], want_logits=False)      # warm the prefill path (buffers, kernel attributes), then start over
            torch.cuda.synchronize()
            eng.dm.check_error()
            eng.reset(0)
        pe0.record()
        eng.prefill(0, ctx, want_logits=True)
        pe1.record()
    first_try.attempt(fill_context)
    try:
        first_try.sync_point()
    except RuntimeError as ex:
        if not token_major:
            raise
        # the headline is the decode step: fill the context through the row-batched path instead and say so
        prefill_note = f"token-major prefill failed ({str(ex)[:160]}); context filled by the row-batched path"
        log(prefill_note)
        torch.cuda.synchronize()
        eng.dm.err_word.zero_()
        eng.tp_channels = None
        eng.opts.prefill_chunk = 0
        token_major = False
        eng.reset(0)
        pe0.record()
        eng.prefill(0, ctx, want_logits=True)
        pe1.record()
        torch.cuda.synchronize()
        eng.dm.check_error()
    prefill_ms = pe0.elapsed_time(pe1)
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
    # the extras run under a lock-step guard: a failure that shows on some ranks only (a bounded wait that ran out) is
    # spread to all ranks at the next sync point, so that their collectives never get out of step
    guard = Lockstep(dist, dev, check=eng.dm.check_error, sync=torch.cuda.synchronize)
    attempt, sync_point = guard.attempt, guard.sync_point

    def run_long_prefill():
        # ---- long prompt: 32,768 tokens in 4,096-token chunks through the token-major path
        prefill_long = None
        if args.prefill_long and token_major:
            lg = torch.Generator().manual_seed(77)
            long_toks = torch.randint(0, cfg.vocab, (args.prefill_long,), generator=lg).tolist()
            eng.reset(1)
            sync_point()
            q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            q0.record()
            attempt(lambda: eng.prefill(1, long_toks, want_logits=True))
            q1.record()
            sync_point()
            tl = torch.tensor([q0.elapsed_time(q1)], device=dev)
            if dist is not None:
                dist.all_reduce(tl, op=dist.ReduceOp.MAX)
            prefill_long = {"tokens": args.prefill_long, "chunk": eng.prefiller.T, "lanes": eng.prefiller.lanes, "ms": round(float(tl), 1),
                            "tok_s": round(args.prefill_long / (float(tl) / 1e3), 1)}
            log(f"long prefill: {prefill_long}")
            eng.reset(1)
        return prefill_long

    def run_mtp():
        # ---- speculative decoding through Session.generate: 5 drafts per step, sampling (T 1.0, top-k 20, top-p 0.95), 1 and 4
        # concurrent streams of 8,192-token context.  Random weights accept next to nothing, so acceptance is forced: for
        # a = 0..5 exactly `a` drafts are accepted per stream and step, and every figure is a timed run of real steps
        # (drafts, one verification step over all streams' rows, sampling of every row, accept / rollback).
        mtp = None
        if args.mtp_context and eng.mtp and (world == 1 or args.comm == "p2p"):
            from qwb200.engine.sampling import SamplingParams
            from qwb200.session.session import Session, StepReq
            ses = attempt(lambda: Session(eng, host_cache_bytes=0))
            sync_point()          # the ranks' hosts leave the set-up together
            kd, steps_m = 5, max(3, args.mtp_steps)
            sp = SamplingParams(temperature=1.0, top_k=20, top_p=0.95, seed=1234)
            mg = torch.Generator().manual_seed(99)
            for sl_ in range(4):
                toks_ = torch.randint(0, cfg.vocab, (args.mtp_context,), generator=mg).tolist()

                def fill(sl_=sl_, toks_=toks_):
                    eng.reset(sl_)
                    ses.sampler.reset_slot(sl_)
                    eng.prefill(sl_, toks_, want_logits=True)
                attempt(fill)
            sync_point()
            mtp = {"drafts": kd, "context": args.mtp_context, "sampling": {"temperature": 1.0, "top_k": 20, "top_p": 0.95},
                   "timed_steps_per_point": steps_m, "note": "measured: forced acceptance of a drafts per stream and step"}
            for streams in (1, 4):
                pend = [7 + i for i in range(streams)]
                res = []
                for acc in range(kd + 1):
                    def one_step():
                        outs = ses.generate([StepReq(i, pend[i], 64, 0, sp) for i in range(streams)], kd, force_accept=acc)
                        for i, o in enumerate(outs):
                            pend[i] = o.tokens[-1]
                        return sum(len(o.tokens) for o in outs)
                    for _ in range(3):
                        attempt(one_step)
                    sync_point()
                    m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    m0.record()
                    emitted = 0
                    for _ in range(steps_m):
                        emitted += attempt(one_step, 0)
                    m1.record()
                    sync_point()
                    tm = torch.tensor([m0.elapsed_time(m1)], device=dev)
                    if dist is not None:
                        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
                    res.append({"accepted": acc, "ms_per_step": round(float(tm) / steps_m, 3), "tok_s": round(emitted / (float(tm) / 1e3), 1)})
                mtp[f"streams_{streams}"] = res
                log(f"speculative, {streams} stream(s): {res}")
        return mtp

    # the headline's times as the maximum over the ranks, taken while the ranks are certainly in step
    if dist is not None:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(tt[0]), float(tt[1])
    # the extras must not take the headline with them: a failure is recorded in their place
    extras_failed = {}
    prefill_long = mtp = None
    for name, fn in (("prefill_long", run_long_prefill), ("mtp", run_mtp)):
        if extras_failed:
            extras_failed[name] = "skipped after an earlier failure"
            continue
        try:
            r = fn()
        except Exception as ex:          # noqa: BLE001 - reported in the JSON line
            r = None
            extras_failed[name] = f"{type(ex).__name__}: {str(ex)[:200]}"
            log(f"{name} failed: {extras_failed[name]}")
            try:
                torch.cuda.synchronize()
                eng.dm.err_word.zero_()
            except Exception:
                pass
        if name == "prefill_long":
            prefill_long = r
        else:
            mtp = r
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
            "prefill_long": prefill_long,
            "mtp": mtp,
            "gpu_launches": launches * K,
            "gpu_launches_per_step": launches,
            "impl": "ours",
        }
        if prefill_note:
            out["prefill"]["note"] = prefill_note
        if extras_failed:
            out["extras_failed"] = extras_failed
        print(json.dumps(out), flush=True)
    if extras_failed:
        # ranks may be out of step after a failure: leave without the collective tear-down (which waits for all of them)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
