"""Does a slot configuration load and run?

    python -m qwb200.tools.slots_probe --slots 6 --max 131072 [--resident 32768] [--fill 4096] [--layers 0]

Builds the engine with ``--slots`` slots of ``--max`` tokens (``--resident`` of them per slot in device memory, the rest
as KV spill in pinned host memory; without it everything is resident), prints the device's free memory and what the
state takes, fills every slot with ``--fill`` tokens and decodes one step across all slots (the widest batch the
configuration allows).  (The reference's bench/slots_probe.hip.)"""
import argparse
import dataclasses
import json
import time

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine import device_model as DM
from ..models.config import ModelConfig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=6)
    ap.add_argument("--max", type=int, default=131072)
    ap.add_argument("--resident", type=int, default=0)
    ap.add_argument("--fill", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0)
    a = ap.parse_args()
    cfg = ModelConfig.full()
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    page = DM.KV_PAGE
    cap = (a.max + page - 1) // page * page
    kw = {}
    if a.resident and a.resident < cap:
        res = a.resident // page
        kw = dict(dev_pages=a.slots * res, host_pages=a.slots * (cap // page - res))
    free0, total = torch.cuda.mem_get_info(0)
    t0 = time.time()
    eng = Engine.synthetic(cfg, EngineOptions(slots=a.slots, slot_tokens=cap, use_graphs=True, prefill_chunk=4096, max_rows=max(8, a.slots), **kw),
                           device="cuda:0", ple_rows=1 << 22)
    free1, _ = torch.cuda.mem_get_info(0)
    out = {"slots": a.slots, "slot_tokens": cap, "resident_tokens": a.resident or cap, "build_s": round(time.time() - t0, 1),
           "device_total_gb": round(total / 2**30, 1), "device_free_before_gb": round(free0 / 2**30, 1), "device_free_after_gb": round(free1 / 2**30, 1),
           "memory": eng.memory_plan(), "spill_numa": eng.dm.spill_numa}
    g = torch.Generator().manual_seed(1)
    for s in range(a.slots):
        eng.prefill(s, torch.randint(0, cfg.vocab, (a.fill,), generator=g).tolist(), want_logits=True)
    toks = eng.decode(list(range(a.slots)), [11] * a.slots)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(8):
        toks = eng.decode(list(range(a.slots)), toks)
    e1.record()
    torch.cuda.synchronize()
    eng.dm.check_error()
    out["decode_all_slots_ms"] = round(e0.elapsed_time(e1) / 8, 3)
    out["ok"] = True
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
