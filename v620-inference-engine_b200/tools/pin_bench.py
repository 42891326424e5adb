"""How long pinning host memory takes, and whether it stalls the rest of the process.

    python -m qwb200.tools.pin_bench [--arena-mb 256] [--rounds 4] [--threads 1,2,4] [--busy] [--decode-steps 0]

For each way of getting pinned memory (``cudaHostAlloc`` through torch, ``mmap`` + ``cudaHostRegister`` through the
pinned pool of ``native/src/pinned_pool.hpp``) and each number of pinning threads: seconds per arena, aggregate GB/s, and
meanwhile the latency of a small mmap + touch + munmap on a probe thread (pinning holds the process's memory-map lock:
every thread that maps or faults memory waits behind it).  Then a host -> device -> host copy of one arena per way
(GB/s each direction).  ``--busy`` keeps the GPU running 20 ms kernels during the pins.  ``--decode-steps N`` adds the
serving question: N decode steps of a small engine timed one by one with and without pinning threads in the background
(median, p99, worst step).
(The reference's bench/pin_bench.hip and bench/decode_stall_bench.hip ask the same two questions.)"""
import argparse
import json
import mmap
import statistics
import threading
import time

import torch


def probe_loop(stop, out):
    """Small anonymous mappings made and dropped: their latency is what a thread of the engine sees while another pins."""
    while not stop.is_set():
        t0 = time.perf_counter()
        m = mmap.mmap(-1, 1 << 16)
        m[0] = 1
        m[4096 * 8] = 1
        m.close()
        out.append((time.perf_counter() - t0) * 1e3)
        time.sleep(0.001)


def pin_torch(nbytes):
    return torch.empty(nbytes, dtype=torch.uint8).pin_memory()


def make_pool_pinner(arena_bytes):
    from ..native import host
    def pin(nbytes):
        pool = host.PinnedPool(unit_bytes=arena_bytes, arena_bytes=arena_bytes, standing_units=0, use_cuda=True)
        pool.reserve(1)
        u = pool.get()                     # waits for the background thread to pin the arena
        return pool, u
    return pin


def run_way(name, pin, arena_bytes, rounds, threads):
    lat, hold = [], []
    lock = threading.Lock()

    def work():
        for _ in range(rounds):
            t0 = time.perf_counter()
            h = pin(arena_bytes)
            dt = time.perf_counter() - t0
            with lock:
                lat.append(dt)
                hold.append(h)
    stop, probe = threading.Event(), []
    pt = threading.Thread(target=probe_loop, args=(stop, probe))
    pt.start()
    t0 = time.perf_counter()
    ts = [threading.Thread(target=work) for _ in range(threads)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    wall = time.perf_counter() - t0
    stop.set()
    pt.join()
    first = hold[0]
    res = {"way": name, "threads": threads, "arenas": len(lat), "s_per_arena_median": round(statistics.median(lat), 4),
           "s_per_arena_max": round(max(lat), 4), "gb_s": round(len(lat) * arena_bytes / wall / 1e9, 2),
           "probe_ms_median": round(statistics.median(probe), 3) if probe else None, "probe_ms_max": round(max(probe), 3) if probe else None}
    return res, first, hold


def copy_speed(host_tensor, dev):
    d = torch.empty(host_tensor.numel(), dtype=torch.uint8, device=dev)
    out = {}
    for name, fn in (("h2d", lambda: d.copy_(host_tensor, non_blocking=True)), ("d2h", lambda: host_tensor.copy_(d, non_blocking=True))):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name + "_gb_s"] = round(4 * host_tensor.numel() / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1)
    return out


def busy_loop(stop, dev):
    a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    s = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(s):
        while not stop.is_set():
            for _ in range(8):
                a @ a
            s.synchronize()


def decode_stall(steps, arena_bytes, threads, dev):
    """Decode steps timed one by one: alone, then with `threads` threads pinning and freeing arenas."""
    import dataclasses
    from ..engine.engine import Engine, EngineOptions
    from ..models.config import ModelConfig
    cfg = dataclasses.replace(ModelConfig.full(), n_layers=4, layer_types=("gdn", "gdn", "gdn", "qsa"))
    eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=4096, use_graphs=True), device=dev, ple_rows=1 << 16)
    eng.prefill(0, list(range(5, 517)))
    tok = 11
    for _ in range(8):                     # graph capture and first-use costs stay out of the timed steps
        tok = eng.decode([0], [tok])[0]
    rows = []

    def run(label, n_pin):
        stop = threading.Event()
        pinned = [0]

        def pinner():
            while not stop.is_set():
                t = pin_torch(arena_bytes)
                pinned[0] += 1
                del t
        ts = [threading.Thread(target=pinner) for _ in range(n_pin)]
        [t.start() for t in ts]
        tok, ms = 11, []
        for _ in range(steps):
            t0 = time.perf_counter()
            tok = eng.decode([0], [tok])[0]
            ms.append((time.perf_counter() - t0) * 1e3)
        stop.set()
        [t.join() for t in ts]
        ms.sort()
        rows.append({"case": label, "median_ms": round(ms[len(ms) // 2], 3), "p99_ms": round(ms[int(len(ms) * 0.99) - 1], 3),
                     "worst_ms": round(ms[-1], 3), "arenas_pinned": pinned[0]})
    run("no pinning", 0)
    run(f"{threads} threads pinning", threads)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arena-mb", type=int, default=256)
    ap.add_argument("--rounds", type=int, default=4)
    ap.add_argument("--threads", default="1,2,4")
    ap.add_argument("--busy", action="store_true")
    ap.add_argument("--decode-steps", type=int, default=0)
    a = ap.parse_args()
    dev = "cuda:0"
    torch.cuda.init()
    torch.zeros(1, device=dev)
    arena = a.arena_mb << 20
    stop = threading.Event()
    bt = None
    if a.busy:
        bt = threading.Thread(target=busy_loop, args=(stop, dev))
        bt.start()
    out = {"arena_mb": a.arena_mb, "busy": a.busy, "rows": [], "copies": {}}
    ways = [("cudaHostAlloc (torch)", pin_torch), ("mmap + cudaHostRegister (pinned pool)", make_pool_pinner(arena))]
    for name, pin in ways:
        for th in [int(x) for x in a.threads.split(",")]:
            res, first, hold = run_way(name, pin, arena, a.rounds, th)
            out["rows"].append(res)
            if name not in out["copies"]:
                t = first if isinstance(first, torch.Tensor) else torch.from_numpy(first[1])
                out["copies"][name] = copy_speed(t, dev)
            del first, hold
    stop.set()
    if bt:
        bt.join()
    if a.decode_steps:
        out["decode_stall"] = decode_stall(a.decode_steps, arena, 4, dev)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
