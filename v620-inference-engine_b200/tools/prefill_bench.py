"""Prefill throughput and where the time goes: tokens per second of one prompt through the token-major path, and the
share of the mixers, attention blocks (GDN / QSA), MoE blocks and the rest, measured with CUDA events around the
Prefiller's phases (a second, instrumented pass; the throughput figure comes from the plain pass).

    python -m qwb200.tools.prefill_bench [--tokens 4096] [--chunk 4096] [--ctx 0] [--layers 0]

(The reference's tool: bench/prefill_bench with --ctx / --tokens-file.)"""
import argparse
import collections
import json

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine.prefill import Prefiller
from ..models.config import ModelConfig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--ctx", type=int, default=0, help="tokens already in the slot before the measured prompt")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--by-kernel", action="store_true", help="a third pass that times every launcher call of the library by name")
    a = ap.parse_args()
    cfg = ModelConfig.full()
    if a.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=a.ctx + 2 * a.tokens + 512, use_graphs=False, prefill_chunk=a.chunk),
                           device="cuda:0", ple_rows=1 << 20)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab, (a.ctx + a.tokens,), generator=g).tolist()
    eng.prefill(0, toks[:512], want_logits=False)          # warm-up
    torch.cuda.synchronize()
    eng.reset(0)
    if a.ctx:
        eng.prefill(0, toks[:a.ctx], want_logits=False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.prefill(0, toks[a.ctx:], want_logits=True)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(f"prefill of {a.tokens} tokens after {a.ctx}: {ms:.1f} ms, {a.tokens / ms * 1e3:.0f} tok/s", flush=True)
    # instrumented pass
    acc = collections.defaultdict(float)
    P = eng.prefiller

    def wrap(name, key_of=lambda *args: None):
        fn = getattr(P, name)

        def timed(*args, **kw):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            r = fn(*args, **kw)
            s1.record()
            torch.cuda.synchronize()
            acc[key_of(*args) or name] += s0.elapsed_time(s1)
            return r
        setattr(P, name, timed)
    wrap("mix")
    wrap("attn_block", lambda lw, *rest: "attn_qsa" if lw["is_qsa"] else "attn_gdn")
    wrap("moe")
    if hasattr(P, "mtp_pass"):
        wrap("mtp_pass")
    eng.reset(0)
    if a.ctx:
        eng.prefill(0, toks[:a.ctx], want_logits=False)
        acc.clear()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    eng.prefill(0, toks[a.ctx:], want_logits=True)
    t1.record()
    torch.cuda.synchronize()
    total = t0.elapsed_time(t1)
    acc["other (embed, PLE, final mix, lm_head, host)"] = total - sum(acc.values())
    for k, v in sorted(acc.items(), key=lambda kv: -kv[1]):
        print(f"  {k:46s} {v:8.1f} ms  {100 * v / total:5.1f} %")
    print(json.dumps({"tokens": a.tokens, "ctx": a.ctx, "ms": round(ms, 1), "tok_s": round(a.tokens / ms * 1e3), "split_ms": {k: round(v, 1) for k, v in acc.items()}}))
    if a.by_kernel:
        by = collections.defaultdict(float)
        n_calls = collections.Counter()

        class TimedLib:
            """Every ``qwk_*`` launcher of the library, bracketed by CUDA events and a synchronize."""
            def __init__(self, lib):
                self._lib = lib

            def __getattr__(self, name):
                fn = getattr(self._lib, name)
                if not name.startswith("qwk_"):
                    return fn

                def timed(*args):
                    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s0.record()
                    r = fn(*args)
                    s1.record()
                    torch.cuda.synchronize()
                    by[name] += s0.elapsed_time(s1)
                    n_calls[name] += 1
                    return r
                return timed
        real = P.lib
        P.lib = TimedLib(real)
        eng.reset(0)
        if a.ctx:
            eng.prefill(0, toks[:a.ctx], want_logits=False)
            by.clear()
            n_calls.clear()
        eng.prefill(0, toks[a.ctx:], want_logits=True)
        P.lib = real
        for k, v in sorted(by.items(), key=lambda kv: -kv[1]):
            print(f"  {k:34s} {n_calls[k]:5d} calls {v:8.1f} ms")


if __name__ == "__main__":
    main()
