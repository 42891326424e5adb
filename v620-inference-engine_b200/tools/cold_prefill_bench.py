"""A long prompt prefilled cold through the Session under different block-store settings, alternating in one process:

    python -m qwb200.tools.cold_prefill_bench [--tokens 65536] [--reps 2] [--host-gb 48] [--configs nostore,ram,ram+disk]

What the saves of the prefix cache cost a prefill: the same prompt with no store at all is the floor.  Every run builds
a new Session (its pinned pool starts empty, as after a restart).  Per run: seconds, tok/s, the pool's arenas pinned
and how long that took, saves that waited for a pinned unit and for how long, bytes the cache holds, and the GPU's
energy for the run (kJ, NVML power integrated over the run).
(The reference's bench/cold_prefill_bench.hip: same question, its configs name pinning strategies of its pools.)"""
import argparse
import dataclasses
import json
import tempfile
import time

import torch

from ..engine.engine import Engine, EngineOptions
from ..models.config import ModelConfig
from ..session.session import Session
from ..utils.power import PowerMeter


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--host-gb", type=float, default=48.0)
    ap.add_argument("--configs", default="nostore,ram,ram+disk")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--piece", type=int, default=4096)
    a = ap.parse_args()
    cfg = ModelConfig.full()
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    cap = (a.tokens + 4096 + 255) // 256 * 256
    eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=cap, use_graphs=True, prefill_chunk=4096), device="cuda:0", ple_rows=1 << 22)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab, (a.tokens,), generator=g).tolist()
    eng.prefill(0, prompt[:4096], want_logits=False)          # warm-up: graphs, attributes, workspaces
    eng.reset(0)
    rows = []
    for rep in range(a.reps):
        for name in a.configs.split(","):
            tmp = tempfile.TemporaryDirectory() if "disk" in name else None
            ses = Session(eng, host_cache_bytes=0 if name == "nostore" else int(a.host_gb * (1 << 30)),
                          disk_cache_dir=tmp.name if tmp else None, disk_cache_bytes=(64 << 30) if tmp else 0, prefill_piece=a.piece)
            eng.reset(0)
            ses.slots[0].busy = True
            torch.cuda.synchronize()
            pm = PowerMeter(indices=[0]).start()
            t0 = time.time()
            ses.begin_prompt(0, prompt)
            while not ses.prefill_some(0, a.piece):
                pass
            torch.cuda.synchronize()
            dt = time.time() - t0
            en = pm.stop()
            tm = ses.slot_timing(0)
            pool = ses.pool.stats() if ses.pool is not None else {}
            st = ses.cache_stats()
            rows.append({"config": name, "rep": rep, "seconds": round(dt, 3), "tok_s": round(a.tokens / dt), "save_s": round(tm["save_s"], 3),
                         "pin_wait_s": round(tm["pin_wait_s"], 3), "arenas": pool.get("arenas"), "pin_seconds": round(pool.get("pin_seconds", 0.0), 3),
                         "unit_waits": pool.get("waits"), "cache_ram_bytes": max(0, int(st.get("ram_bytes") or 0)) if name != "nostore" else 0, "cache_disk_bytes": st.get("disk_bytes"), "kilojoules": en.get("kilojoules"),
                         "avg_w": en.get("avg_w")})
            print(json.dumps(rows[-1]), flush=True)
            ses.slots[0].busy = False
            del ses
            if tmp:
                tmp.cleanup()
    eng.dm.check_error()


if __name__ == "__main__":
    main()
