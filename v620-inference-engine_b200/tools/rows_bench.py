"""Milliseconds per batched decode step at 1 / 2 / 4 / 8 ... rows (CUDA-graph replay, CUDA events), plain and with
the speculative-verification flags (GDN state saved after every row, hidden states kept):

    python -m qwb200.tools.rows_bench [--rows 1,2,4,8,16] [--layers 0] [--context 1024] [--slots 1|rows]

``--slots rows`` gives every row its own sequence (independent streams); the default runs the rows as one run of a
single sequence, which is what verification does.  (The reference publishes 14.73 / 16.60 / 21.03 / 26.42 ms at
1 / 2 / 4 / 8 rows on its four cards.)"""
import argparse
import json

import torch

from ..engine import device_model as DM
from ..engine.engine import Engine, EngineOptions
from ..models.config import ModelConfig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="1,2,4,8")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--slots", default="1")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--profile", action="store_true", help="bracket one extra step per row count with cudaProfilerStart/Stop")
    a = ap.parse_args()
    rows = [int(x) for x in a.rows.split(",")]
    cfg = ModelConfig.full()
    if a.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    per_row = a.slots == "rows"
    n_slots = max(rows) if per_row else 1
    eng = Engine.synthetic(cfg, EngineOptions(slots=n_slots, slot_tokens=a.context + 64 * a.reps * 2 + 256, use_graphs=True, save_gdn=True),
                           device="cuda:0", ple_rows=1 << 20)
    g = torch.Generator().manual_seed(1)
    ctx = torch.randint(0, cfg.vocab, (a.context,), generator=g).tolist()
    for s in range(n_slots):
        eng.prefill(s, ctx, want_logits=False)
    out = {}
    for M in rows:
        for name, flags in (("plain", 0), ("verify", DM.FLAG_SAVE_GDN | DM.FLAG_KEEP_HIDDEN)):
            def step():
                if per_row:
                    sl, base = list(range(M)), [eng.slot[s].n for s in range(M)]
                    pos = base
                else:
                    sl, pos = [0] * M, list(range(eng.slot[0].n, eng.slot[0].n + M))
                toks = [5 + i for i in range(M)]
                eng.dm.step(toks, sl, pos, eng._ctx3(0, toks), flags=flags, graph=True)
                for s_, t in zip(sl, toks):
                    eng.slot[s_].tokens.append(t)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.reps):
                step()
            e1.record()
            torch.cuda.synchronize()
            if a.profile and name == "plain":
                torch.cuda.profiler.start()
                step()
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
            out[f"{name}_{M}"] = round(e0.elapsed_time(e1) / a.reps, 3)
            print(f"rows={M:2d} {name:6s}: {out[f'{name}_{M}']:.3f} ms per step, {M / out[f'{name}_{M}'] * 1e3:.0f} tok/s", flush=True)
    eng.dm.check_error()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
