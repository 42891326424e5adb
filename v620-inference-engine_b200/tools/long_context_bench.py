"""Long-context serving measurements on one GPU: KV spill, the shared-prefix restore and the n-gram table gather.

    python -m qwb200.tools.long_context_bench [--slots 6] [--tokens 131072] [--resident 32768] [--prefix 12288]
                                              [--ple-gb 4] [--decode-steps 32] [--layers 0]

Every slot holds ``--tokens`` tokens of context of which the first ``--resident`` live in device memory and the rest
in pinned host memory that the attention kernels read directly (a deliberately small device quota: on this GPU the whole
context would fit).  Reported:

* prefill tokens per second into the resident part and into the spilled part of a slot;
* decode milliseconds per step for a row whose context is all resident against a row whose selected tokens lie mostly
  in host memory, with the device cache in front of the host pages (its hit rate) and without it;
* seconds to restore a ``--prefix``-token shared prefix from the host block store into a second slot, against
  prefilling it;
* gigabytes per second of the fp8 n-gram table gather (16 rows per token) from a pinned host table of ``--ple-gb`` GB.

(The reference's tools: bench/spill_bench, bench/spill_gather_bench, bench/prefix_cache_bench.)"""
import argparse
import ctypes as C
import dataclasses
import json
import time

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine import device_model as DM
from ..models.config import ModelConfig
from ..session.session import Session
from ..utils import settings


def timed(fn):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), (time.time() - t0) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=6)
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--resident", type=int, default=32768)
    ap.add_argument("--prefix", type=int, default=12288)
    ap.add_argument("--ple-gb", type=float, default=4.0)
    ap.add_argument("--decode-steps", type=int, default=32)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--filled", type=int, default=2, help="slots that are actually filled with --tokens tokens (the others only reserve memory)")
    ap.add_argument("--cache-mb", type=int, default=256)
    a = ap.parse_args()
    cfg = ModelConfig.full()
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    settings.set_current(settings.Settings.from_env(spill_cache_mb=a.cache_mb, spill_cache_stats=True))
    page = DM.KV_PAGE
    cap = (a.tokens + 2 * a.decode_steps + 4096 + page - 1) // page * page
    res_pages = a.resident // page
    max_pages = cap // page
    ple_rows = int(a.ple_gb * (1 << 30) / cfg.ngram_dim)
    opts = EngineOptions(slots=a.slots, slot_tokens=cap, use_graphs=True, prefill_chunk=4096, dev_pages=a.slots * res_pages,
                         host_pages=a.slots * (max_pages - res_pages))
    t0 = time.time()
    eng = Engine.synthetic(cfg, opts, device="cuda:0", ple_rows=ple_rows)
    out = {"slots": a.slots, "tokens": a.tokens, "resident": a.resident, "layers": cfg.n_layers,
           "host_kv_gb": round(sum(t.numel() * 2 for t in (eng.dm.k_host or []) + (eng.dm.v_host or [])) / 2**30, 2),
           "ple_table_gb": round(ple_rows * cfg.ngram_dim / 2**30, 2), "build_s": round(time.time() - t0, 1)}
    out["spill_numa"] = eng.dm.spill_numa
    g = torch.Generator().manual_seed(5)
    ctx = [torch.randint(0, cfg.vocab, (a.tokens,), generator=g).tolist() for _ in range(a.filled)]
    eng.prefill(0, ctx[0][:512], want_logits=False)          # warm-up
    eng.reset(0)
    # ---- prefill: resident part, then spilled part
    ms_res, _ = timed(lambda: eng.prefill(0, ctx[0][:a.resident], want_logits=False))
    ms_sp, _ = timed(lambda: eng.prefill(0, ctx[0][a.resident:], want_logits=True))
    out["prefill_resident_tok_s"] = round(a.resident / ms_res * 1e3)
    out["prefill_spilled_tok_s"] = round((a.tokens - a.resident) / ms_sp * 1e3)
    for s in range(1, a.filled):
        eng.prefill(s, ctx[s], want_logits=True)
    eng.dm.check_error()
    # ---- decode: a short all-resident slot against the long, mostly spilled one
    short = a.slots - 1
    eng.prefill(short, ctx[0][:min(a.resident, 8192)], want_logits=True)

    def decode_ms(slot, steps):
        t = 11
        for _ in range(4):
            t = eng.decode([slot], [t])[0]
        ms, _ = timed(lambda: [eng.decode([slot], [t]) for _ in range(steps)])
        return ms / steps
    out["decode_ms_resident_row"] = round(decode_ms(short, a.decode_steps), 3)
    st0 = eng.dm.spill_cache_stats()
    out["decode_ms_spilled_row"] = round(decode_ms(0, a.decode_steps), 3)
    st1 = eng.dm.spill_cache_stats()
    if st0 and st1:
        h, m = st1[0] - st0[0], st1[1] - st0[1]
        out["spill_cache_hit_rate"] = round(h / max(1, h + m), 3)
    out["decode_ms_per_spilled_row_extra"] = round(out["decode_ms_spilled_row"] - out["decode_ms_resident_row"], 3)
    # ---- shared prefix: save through the session's block store, restore into another slot
    ses = Session(eng, host_cache_bytes=64 << 30, prefill_piece=2048)
    prefix = ctx[0][:a.prefix]
    pa = prefix + [5, 6, 7]
    sa = a.slots - 2
    eng.reset(sa)
    ses.slots[sa].busy = True
    t1 = time.time()
    ses.begin_prompt(sa, pa)
    while not ses.prefill_some(sa, 2048):
        pass
    torch.cuda.synchronize()
    out["prefix_cold_s"] = round(time.time() - t1, 3)
    out["prefix_save_s"] = round(ses.slots[sa].timing["save_s"], 3)
    out["prefix_pin_wait_s"] = round(ses.slots[sa].timing["pin_wait_s"], 3)
    sb = a.slots - 3 if a.slots >= 4 else short
    eng.reset(sb)
    ses.slots[sb].busy = True
    pb = prefix + [9, 8, 7, 6]
    t2 = time.time()
    reused = ses.begin_prompt(sb, pb)
    torch.cuda.synchronize()
    out["prefix_restore_s"] = round(time.time() - t2, 3)
    out["prefix_restored_tokens"] = int(reused)
    while not ses.prefill_some(sb, 2048):
        pass
    torch.cuda.synchronize()
    out["prefix_warm_total_s"] = round(time.time() - t2, 3)
    # ---- n-gram table gather from pinned host memory
    T = 4096
    dm = eng.dm
    ctx3 = torch.randint(0, cfg.vocab, (T, 3), generator=g, dtype=torch.int32).to(dm.dev)
    e_out = torch.zeros(T, cfg.hidden, dtype=torch.bfloat16, device=dm.dev)
    p = dm.model.ple
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: dm.lib.qwk_ple_gather(C.c_void_p(ctx3.data_ptr()), C.c_void_p(p.shards), C.c_void_p(p.scales), p.rows_per_shard, p.rows,
                                         p.layout, cfg.ngram_dim, cfg.ngram_heads, C.c_void_p(e_out.data_ptr()), None, T, s)
    call()
    ms_g, _ = timed(lambda: [call() for _ in range(10)])
    out["ple_gather_gb_s"] = round(10 * T * cfg.ngram_heads * cfg.ngram_dim / (ms_g * 1e-3) / 1e9, 1)
    eng.dm.check_error()
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
