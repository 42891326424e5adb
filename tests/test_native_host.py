"""Native host runtime (C++): hasher, PLE table, block store + disk tier, sampler, chunker."""
import os
import struct
import time

import numpy as np
import pytest
import torch

from qwb200.models.config import ModelConfig
from qwb200.models.ngram import NgramHasher as PyHasher
from qwb200.models.ple import PleTable
from qwb200.native import host as H


def test_native_hasher_equals_python():
    for cfg in (ModelConfig.full(), ModelConfig.tiny()):
        a, b = H.NgramHasher(cfg), PyHasher(cfg)
        assert a.total_rows == b.total_rows
        toks = [7, 9, cfg.eos, 3, 3, cfg.eos, cfg.eos, 12, -3, 5, cfg.vocab - 1]
        assert np.array_equal(a.ids_for([], toks), b.ids_for([], toks))
        assert np.array_equal(a.ids_for(toks[:4], toks[4:]), b.ids_for(toks[:4], toks[4:]))


@pytest.mark.parametrize("layout", ["f8", "bf16", "int8", "int4"])
def test_native_ple_table_equals_python(tmp_path, layout):
    cfg = ModelConfig.tiny()
    t = PleTable.synthetic(cfg, rows=777, layout=layout, n_shards=2, seed=3)
    t.save(str(tmp_path))
    nat = H.PleTableNative(str(tmp_path), cfg.ngram_dim, threads=3)
    ids = np.random.default_rng(0).integers(0, 5000, size=(40, cfg.ngram_heads))
    want = t.gather(ids).numpy()
    got = nat.gather(ids)
    assert np.allclose(got, want, rtol=0, atol=1e-6)


def test_block_store_chain_restore_and_disk_format(tmp_path):
    layout = 0x1234
    st = H.BlockStore(layout, 2, ram_budget=1 << 20, disk_dir=str(tmp_path), disk_budget=1 << 22)
    toks = list(range(1000, 1000 + 600))
    parent, keys = st.root, []
    for i in range(0, 600, 256):
        blk = toks[i:i + 256]
        k = st.save_block(parent, i, blk, bytes([i // 256 + 1]) * 1000)
        assert k == H.BlockStore.key(parent, blk) and k != 0
        keys.append(k)
        parent = k
    assert st.save_snapshot(keys[1], b"S" * 500, np.arange(5, dtype=np.float32), anchor=True)
    path, depth = st.lookup(toks)
    assert path == keys and depth == 2
    path, depth = st.lookup(toks[:300] + [1, 2, 3])
    assert path == keys[:1] and depth == 0
    snap, lg = st.get(keys[1], snapshot=True)
    assert snap == b"S" * 500 and lg.tolist() == [0, 1, 2, 3, 4]
    assert st.get(keys[2]) == bytes([3]) * 1000
    st.flush()
    # file format: header | tokens | logits | payload
    f = os.path.join(str(tmp_path), f"{keys[0]:016x}.qwb")
    raw = open(f, "rb").read()
    magic, lay, h, par, ntok, ranks, nlog, rb = struct.unpack("<8sQQQqIIQ", raw[:56])
    assert magic == b"QWBLOCK2" and lay == layout and h == keys[0] and par == st.root and ntok == 256 and ranks == 2
    assert nlog == 0 and rb == 500 and len(raw) == 56 + 256 * 4 + 1000
    assert struct.unpack("<256i", raw[56:56 + 1024]) == tuple(toks[:256])
    s = open(os.path.join(str(tmp_path), f"{keys[1]:016x}.qws"), "rb").read()
    assert s[:8] == b"QWSNAPS1" and len(s) == 56 + 5 * 4 + 500
    stats = st.stats()
    assert stats["blocks"] == 3 and stats["snapshots"] == 1 and stats["disk_bytes"] > 0
    st.close()
    # a new store rebuilds its index from the files and serves payloads from disk
    st2 = H.BlockStore(layout, 2, ram_budget=1 << 20, disk_dir=str(tmp_path), disk_budget=1 << 22)
    path, depth = st2.lookup(toks)
    assert path == keys and depth == 2
    assert st2.info(keys[0]) == {"start": 0, "ntok": 256, "has_snap": False, "in_ram": False, "on_disk": True}
    assert st2.info(keys[2])["start"] == 512
    assert st2.get(keys[0]) == bytes([1]) * 1000
    st2.close()
    # another layout id: files are unusable and dropped
    st3 = H.BlockStore(layout + 1, 2, ram_budget=1 << 20, disk_dir=str(tmp_path), disk_budget=1 << 22)
    assert st3.lookup(toks)[0] == [] and not any(n.endswith(".qwb") for n in os.listdir(str(tmp_path)))
    st3.close()


def test_block_store_truncated_file_is_dropped(tmp_path):
    st = H.BlockStore(7, 1, 1 << 20, str(tmp_path), 1 << 22)
    k = st.save_block(st.root, 0, list(range(256)), b"x" * 4096)
    st.flush()
    st.close()
    f = os.path.join(str(tmp_path), f"{k:016x}.qwb")
    data = open(f, "rb").read()
    open(f, "wb").write(data[:200])                       # fault injection: a cut-off write
    st2 = H.BlockStore(7, 1, 1 << 20, str(tmp_path), 1 << 22)
    assert st2.lookup(list(range(256)))[0] == [] and not os.path.exists(f)
    st2.close()


def test_block_store_ram_budget_evicts_lru_without_disk():
    st = H.BlockStore(1, 1, ram_budget=2500, disk_dir=None)
    a = st.save_block(st.root, 0, [1] * 256, b"a" * 1000)
    b = st.save_block(st.root, 0, [2] * 256, b"b" * 1000)
    st.lookup([1] * 256)                                  # touch a
    c = st.save_block(st.root, 0, [3] * 256, b"c" * 1000)
    assert st.get(b) is None and st.get(a) is not None and st.get(c) is not None
    assert st.stats()["ram_bytes"] <= 2500


def test_sampler_greedy_penalties_and_distribution():
    s = H.HostSampler(seed=1)
    logits = np.array([0.1, 2.0, 1.9, -1.0, 0.5], dtype=np.float32)
    tok, lp = s.sample(logits, H.Sampling.make())
    assert tok == 1 and abs(lp - (2.0 - np.log(np.exp(logits.astype(np.float64)).sum()))) < 1e-5
    # repetition + presence penalties move the argmax
    tok, _ = s.sample(logits, H.Sampling.make(repetition_penalty=2.0), hist=[1], prompt_end=0)
    assert tok == 2
    tok, _ = s.sample(logits, H.Sampling.make(presence_penalty=0.5), hist=[1], prompt_end=0)
    assert tok == 2
    tok, _ = s.sample(logits, H.Sampling.make(presence_penalty=0.5), hist=[1], prompt_end=1)     # prompt tokens do not count
    assert tok == 1
    # top-k 2 never leaves the top two; frequencies follow the renormalised softmax
    p = H.Sampling.make(temperature=1.0, top_k=2)
    draws = [s.sample(logits, p)[0] for _ in range(4000)]
    assert set(draws) == {1, 2}
    f1 = draws.count(1) / 4000
    assert abs(f1 - 1 / (1 + np.exp(-0.1))) < 0.03
    # top-p keeps the smallest prefix reaching p; min-p is relative to the best token
    assert {s.sample(logits, H.Sampling.make(temperature=1.0, top_p=0.3))[0] for _ in range(200)} == {1}
    assert {s.sample(logits, H.Sampling.make(temperature=1.0, min_p=0.95))[0] for _ in range(200)} == {1}
    # a fixed seed gives the same token for the same history length
    p = H.Sampling.make(temperature=1.0, seed=42)
    assert len({s.sample(logits, p, hist=[0, 0, 0])[0] for _ in range(20)}) == 1
    ids, lps = H.HostSampler.top_logprobs(logits, 3)
    assert ids.tolist() == [1, 2, 4] and lps[0] > lps[1] > lps[2]


def test_chunker_tiles_and_is_position_independent():
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 50000, size=6000).tolist()
    toks[1500] = 99999                                     # a message boundary
    ch = H.chunk_prompt(toks, 99999)
    assert ch[0][0] == 0 and sum(c[1] for c in ch) == len(toks)
    assert all(a[0] + a[1] == b[0] for a, b in zip(ch, ch[1:]))
    assert any(c[0] == 1500 for c in ch) and all(c[1] <= 2048 for c in ch)
    # content-defined: the same text after a different prefix soon falls back into the same chunks
    ch2 = H.chunk_prompt(rng.integers(0, 50000, size=333).tolist() + toks, 99999)
    assert len({c[2] for c in ch} & {c[2] for c in ch2}) >= len(ch) - 3


def test_pinned_pool_units_reserve_retire_and_wait_accounting():
    import threading
    import time
    from qwb200.native import host as H
    unit = 1 << 20
    pool = H.PinnedPool(unit, arena_bytes=4 << 20, standing_units=2, policy="preferred", node=0)
    assert pool.unit_bytes == unit and H.numa_nodes() >= 1
    held = [pool.get() for _ in range(6)]                  # more than one arena of 4 units
    for i, a in enumerate(held):
        a[:] = i                                           # units are distinct, writable memory
    assert [int(a[0]) for a in held] == list(range(6)) and [int(a[-1]) for a in held] == list(range(6))
    st = pool.stats()
    assert st["arenas"] >= 2 and st["gets"] == 6 and st["units_total"] == 4 * st["arenas"]
    for a in held:
        pool.put(a)
    time.sleep(0.3)                                        # the worker retires arenas beyond the standing reserve
    st2 = pool.stats()
    assert 1 <= st2["arenas"] <= st["arenas"] and st2["units_free"] >= 2
    # a consumer blocked on an empty pool is served when a unit comes back
    small = H.PinnedPool(4096, arena_bytes=4096, standing_units=1)
    a = small.get()
    got = []
    t = threading.Thread(target=lambda: got.append(small.get()))
    t.start()
    t.join(timeout=5)                                      # a second arena is made for it (pool grows on demand)
    assert got and got[0].ctypes.data != a.ctypes.data
    assert small.stats()["waits"] >= 1
    small.put(a)
    small.put(got[0])
    with pytest.raises(KeyError):
        small.put(np.zeros(4096, np.uint8))                # not one of this pool's units
    pool.close()
    small.close()


def test_block_store_prefetch_loads_disk_blocks_in_the_background(tmp_path):
    """After a restart the index knows the blocks but their payloads are only on disk; ``prefetch`` queues reads on the
    loader thread and ``loads_pending`` drops to zero with the payloads (and the last snapshot) back in RAM."""
    import time
    st = H.BlockStore(1, 1, 64 << 20, str(tmp_path), 1 << 30)
    toks = list(range(768))
    keys, parent = [], st.root
    for b in range(3):
        parent = st.save_block(parent, b * 256, toks[b * 256:(b + 1) * 256], bytes([65 + b]) * 8192)
        keys.append(parent)
    assert st.save_snapshot(keys[-1], b"s" * 256)
    st.flush()
    del st
    st = H.BlockStore(1, 1, 64 << 20, str(tmp_path), 1 << 30)
    path, depth = st.lookup(toks + [5])
    assert depth == 3 and not any(st.info(k)["in_ram"] for k in path[:3])
    assert st.prefetch(path[:depth]) == 4                  # three KV payloads and the last block's snapshot
    t0 = time.time()
    while st.loads_pending() and time.time() - t0 < 10:
        time.sleep(0.01)
    assert st.loads_pending() == 0 and all(st.info(k)["in_ram"] for k in path[:3])
    assert st.prefetch(path[:depth]) == 0                  # nothing left to read
    assert st.get(path[1]) == bytes([66]) * 8192


def test_block_store_snapshot_by_address_round_trip():
    """Snapshot payloads given and taken by address (the engine's pinned snapshot buffer): same bytes back, a buffer that is
    too small is refused, a block without a snapshot answers -1."""
    st = H.BlockStore(7, 1, 8 << 20)
    toks = list(range(512))
    k0 = st.save_block(st.root, 0, toks[:256], b"k" * 64)
    k1 = st.save_block(k0, 256, toks[256:], b"k" * 64)
    src = (np.arange(5000, dtype=np.uint32) * 2654435761 % 251).astype(np.uint8)
    assert st.save_snapshot_from(k1, src.ctypes.data, src.nbytes, anchor=False)
    out = np.zeros(6000, dtype=np.uint8)
    assert st.get_snapshot_into(k1, out) == 5000 and bytes(out[:5000]) == bytes(src)
    assert st.get_snapshot_into(k1, np.zeros(100, dtype=np.uint8)) == -1
    assert st.get_snapshot_into(k0, out) == -1
    assert st.get(k1, snapshot=True)[0] == bytes(src)


def test_block_store_thins_snapshots_that_crowd_the_next_one(tmp_path):
    """Snapshots closer than the gap to the next kept snapshot further down the conversation are dropped (RAM and file),
    deepest first; anchors, snapshots that were restored from, leaves and branch points stay."""
    st = H.BlockStore(9, 1, ram_budget=1 << 22, disk_dir=str(tmp_path), disk_budget=1 << 24)
    toks = list(range(5000, 5000 + 6 * 256))
    parent, keys = st.root, []
    for i in range(6):
        k = st.save_block(parent, i * 256, toks[i * 256:(i + 1) * 256], bytes([i + 1]) * 512)
        keys.append(k)
        parent = k
        assert st.save_snapshot(k, bytes([65 + i]) * 300, None, anchor=(i == 2))
    st.flush()
    snap_file = lambda k: os.path.join(str(tmp_path), f"{k:016x}.qws")
    assert all(os.path.exists(snap_file(k)) for k in keys)
    # ends 256 512 768* 1024 1280 1536 (the leaf; * = anchor), gap 600: 1280 and 1024 crowd the leaf; 768 is an anchor;
    # 512 is 256 before the anchor -> dropped; 256 is 512 before it -> dropped too
    assert st.thin(600) == 4
    has = [st.info(k)["has_snap"] for k in keys]
    assert has == [False, False, True, False, False, True]
    assert [os.path.exists(snap_file(k)) for k in keys] == has
    assert st.get(keys[3], snapshot=True) is None and st.get(keys[5], snapshot=True)[0] == bytes([70]) * 300
    assert st.get(keys[3]) == bytes([4]) * 512                                   # the blocks themselves are untouched
    assert st.thin(600) == 0                                                      # nothing left to drop
    path, depth = st.lookup(toks + [1])
    assert path == keys and depth == 6                                            # the deepest snapshot still serves the whole prefix
    st.close()
    # a gap smaller than the spacing drops nothing; a branch point is never dropped
    st = H.BlockStore(9, 1, ram_budget=1 << 22, disk_dir=None)
    a = st.save_block(st.root, 0, [1] * 256, b"a" * 64)
    st.save_snapshot(a, b"s" * 32, None, anchor=False)
    b1 = st.save_block(a, 256, [2] * 256, b"b" * 64)
    b2 = st.save_block(a, 256, [3] * 256, b"c" * 64)
    st.save_snapshot(b1, b"t" * 32, None, anchor=False)
    st.save_snapshot(b2, b"u" * 32, None, anchor=False)
    assert st.thin(10000) == 0 and st.info(a)["has_snap"]
    st.close()


def test_thread_pool_visits_every_index_once():
    """The worker pool behind the PLE gather and the fp32 oracle: many short loops back to back (late helpers must not
    disturb the next loop), sizes that do not divide, a grain larger than the loop, one thread."""
    L = H.lib()
    for threads in (1, 2, 8):
        pool = L.qwh_pool_new(threads)
        assert L.qwh_pool_size(pool) == threads
        for n, grain, rounds in ((1, 1, 50), (7, 1, 2000), (1000, 1, 500), (1001, 64, 500), (100, 1000, 50), (100003, 17, 20), (0, 1, 3)):
            assert L.qwh_pool_check(pool, n, grain, rounds) == 0, (threads, n, grain)
        L.qwh_pool_free(pool)


def test_sampler_partial_ordering_equals_the_full_sort():
    """The host sampler orders only as many candidates as a truncation looks at; token and log-probability must equal
    the straightforward form that sorts them all - flat, typical and peaked distributions, ties, every truncation mix."""
    L = H.lib()
    V = 60000
    rng = np.random.default_rng(3)
    cases = [dict(temperature=1.0), dict(temperature=1.0, top_k=20, top_p=0.95), dict(temperature=1.0, top_k=200, top_p=0.9, min_p=0.001),
             dict(temperature=1.0, top_p=0.95), dict(temperature=1.0, top_p=0.9999), dict(temperature=1.3, min_p=0.05),
             dict(temperature=1.0, min_p=1e-9), dict(temperature=0.7, top_p=0.9, min_p=0.01), dict(temperature=1.0, top_k=100000, top_p=0.9),
             dict(temperature=1.0, top_k=20, top_p=0.95, presence_penalty=1.5, repetition_penalty=1.1)]
    try:
        for sigma in (0.3, 3.0, 9.0):
            for trial in range(4):
                logits = (rng.standard_normal(V) * sigma).astype(np.float32)
                if trial == 3:
                    logits[:3000] = logits[0]                     # a plateau of equal logits: ties go to the lower index
                hist = [int(x) for x in rng.integers(0, V, 300)]
                for kw in cases:
                    got = []
                    for full in (1, 0):
                        L.qwh_sampler_full_sort(full)
                        got.append(H.HostSampler(seed=1).sample(logits, H.Sampling.make(seed=50 + trial, **kw), hist=hist, prompt_end=100))
                    assert got[0] == got[1], (sigma, trial, kw, got)
    finally:
        L.qwh_sampler_full_sort(0)


def test_spec_planner_decisions():
    """Native planner of the speculative step: the expected-rate rule, stretches without drafts, limits, acceptance."""
    base, beta = 1.25, 0.25
    pl = H.SpecPlanner(3, base, beta, 0.3, 32, 48, 176)
    for a in (0.0, 0.2, 0.5, 0.8, 0.99):
        for k_max in (1, 2, 5, 12):
            best, bk, expect, p = 0.0, 1, 1.0, 1.0
            for K in range(1, k_max + 1):
                p *= a
                expect += p
                r = expect / (base + beta * (K - 1))
                if r > best:
                    best, bk = r, K
            rate, k = pl.best_rate(a, k_max)
            assert abs(rate - best) < 1e-12 and k == bk
    assert [s.accept for s in pl.slots] == [0.5] * 3 and pl.slots[0].plain_stretch == 32
    # acceptance 0.5 pays with one draft (1.5 / 1.25); 0.1 does not: a stretch starts and the next one will be longer
    assert pl.plan([0], [64], [1000], [True], 4, 12, 0, 32, False) == [1]
    pl.slots[1].accept = 0.1
    assert pl.plan([1], [64], [1000], [True], 4, 12, 0, 32, False) == [0]
    assert (pl.slots[1].plain_left, pl.slots[1].plain_stretch) == (32, 80)
    assert pl.plan([1], [64], [1000], [True], 4, 12, 0, 32, False) == [0] and pl.slots[1].plain_left == 32       # inside the stretch: untouched
    for left in range(31, -1, -1):
        assert pl.note_plain_step(1) == left
    assert abs(pl.slots[1].accept - 0.3) < 1e-12                                      # the stretch is over: the next step probes
    assert pl.plan([1], [64], [1000], [True], 4, 12, 0, 32, False) == [1]
    # forced runs ignore the rule; budget, room, the run limit and the row limit all bind
    assert pl.plan([1, 2], [64, 3], [1000, 1000], [True, True], 5, 12, 0, 32, True) == [5, 2]
    assert pl.plan([1, 2], [64, 64], [2, 1000], [True, False], 5, 12, 4, 32, True) == [2, 0]
    assert pl.plan([0, 1, 2], [64] * 3, [1000] * 3, [True] * 3, 12, 12, 0, 20, True) == [5, 6, 6]      # the first of the longest runs is trimmed first
    import pytest
    with pytest.raises(ValueError, match="budget"):
        pl.plan([0], [0], [10], [True], 4, 12, 0, 32, False)
    with pytest.raises(ValueError, match="slot 2 is full"):
        pl.plan([0, 2], [8, 8], [10, -1], [True, True], 4, 12, 0, 32, False)
    with pytest.raises(ValueError, match="more requests"):
        pl.plan([0, 1, 2], [8] * 3, [10] * 3, [False] * 3, 4, 12, 0, 2, False)
    # acceptance: drafts equal to what was drawn behind them are kept, a stop token ends the run, the average moves by a tenth
    pl.slots[0].accept = 0.5
    assert pl.accept(0, [7, 8, 9, 1], [7, 8, 5], [], None) == 3                        # two drafts kept, the third differs
    assert abs(pl.slots[0].accept - (0.45 + 0.1 * 2 / 3)) < 1e-12
    assert pl.accept(0, [7, 8, 9, 1], [7, 8, 9], [8], None) == 2                        # 8 is a stop token: nothing behind it
    assert pl.accept(0, [7], [], [], None) == 1 and pl.accept(0, [1, 2, 3], [9, 9], [], 5) == 3      # forced: all drafts, at most
    pl.slots[0].plain_stretch = 128
    pl.slots[0].accept = 0.6
    pl.accept(0, [1, 2], [1], [], None)
    assert pl.slots[0].plain_stretch == 32                                            # a good spell resets the stretch length


def test_slot_and_prompt_decisions():
    """Native slot logic: slot choice, the four ways to start a prompt, snapshot choice, capture planning."""
    # most kept, then least recently used; busy and too small slots never
    assert H.choose_slot([False, False, False], [100, 100, 100], [0, 50, 50], [3, 9, 4], 60) == 2
    assert H.choose_slot([False, True, False], [100, 100, 40], [10, 90, 99], [1, 2, 3], 60) == 0
    assert H.choose_slot([True, True], [100, 100], [0, 0], [1, 2], 10) == -1
    # a device snapshot must beat both others; in place wins a tie with the store; nothing to reuse: reset
    assert H.start_way(100, 300, 256) == H.START_DEVICE_SNAPSHOT and H.start_way(300, 300, 256) == H.START_IN_PLACE
    assert H.start_way(256, 0, 256) == H.START_IN_PLACE and H.start_way(100, 200, 512) == H.START_STORE
    assert H.start_way(0, 0, 0) == H.START_RESET and H.start_way(0, 5, 0) == H.START_DEVICE_SNAPSHOT
    # the deepest snapshot inside the common part; one as deep as the prompt only with its logits
    assert H.best_snapshot([100, 300, 500], [False, False, False], 400, 1000) == 1
    assert H.best_snapshot([100, 300], [False, True], 300, 300) == 1 and H.best_snapshot([100, 300], [False, False], 300, 300) == 0
    assert H.best_snapshot([500], [True], 400, 1000) == -1 and H.best_snapshot([0], [True], 10, 20) == -1
    # capture planning against the plain loop
    rng = np.random.default_rng(8)
    for _ in range(300):
        n = int(rng.integers(2, 400))
        prompt = [int(x) for x in rng.integers(0, 6, n)]
        done = int(rng.integers(0, n))
        end = int(rng.integers(done + 1, n + 1))
        last, gap, boundary = int(rng.integers(0, done + 1)), int(rng.integers(1, 60)), 3
        lo, want = max(done + 1, last + gap), end
        for p in range(min(end, n - 1), lo - 1, -1):
            if prompt[p] == boundary:
                want = p
                break
        top = min(end, n - 1)
        assert H.capture_point(prompt[done:top + 1], done, n, done, end, last, boundary, gap) == want
        assert H.capture_point(prompt, 0, n, done, end, last, boundary, gap) == want
        assert H.capture_point(prompt[done:top + 1], done, n, done, end, last, -1, gap) == end


def test_block_store_reads_files_with_the_older_block_magic(tmp_path):
    """A cache directory written with the first block format (magic QWBLOCK1) is indexed and served like the current one."""
    st = H.BlockStore(5, 1, 1 << 20, str(tmp_path), 1 << 22)
    toks = list(range(300, 556))
    k = st.save_block(st.root, 0, toks, b"v" * 777)
    st.flush()
    st.close()
    f = os.path.join(str(tmp_path), f"{k:016x}.qwb")
    raw = bytearray(open(f, "rb").read())
    assert raw[:8] == b"QWBLOCK2"
    raw[:8] = b"QWBLOCK1"
    open(f, "wb").write(bytes(raw))
    st2 = H.BlockStore(5, 1, 1 << 20, str(tmp_path), 1 << 22)
    path, _ = st2.lookup(toks + [1])
    assert path == [k] and st2.get(k) == b"v" * 777
    st2.close()


def test_block_store_concurrent_reads_from_disk(tmp_path):
    """Blocks that live only on disk are read by several threads at once, with background prefetches running: every
    reader gets its block's bytes, nothing deadlocks."""
    import threading
    st = H.BlockStore(6, 1, ram_budget=8 << 10, disk_dir=str(tmp_path), disk_budget=1 << 24)       # RAM holds almost nothing
    parent, keys = st.root, []
    for i in range(24):
        k = st.save_block(parent, i * 256, [1000 * i + j for j in range(256)], bytes([i]) * 4096)
        keys.append(k)
        parent = k
    st.flush()
    st.close()
    st = H.BlockStore(6, 1, ram_budget=8 << 10, disk_dir=str(tmp_path), disk_budget=1 << 24)
    errors = []

    def reader(offset):
        try:
            for rep in range(20):
                i = (offset * 5 + rep * 7) % len(keys)
                got = st.get(keys[i])
                if got != bytes([i]) * 4096:
                    errors.append((offset, i, None if got is None else len(got)))
        except Exception as ex:          # noqa: BLE001
            errors.append((offset, repr(ex)))
    ts = [threading.Thread(target=reader, args=(o,)) for o in range(8)]
    for t in ts:
        t.start()
    st.prefetch(keys[:12], last_snapshot=False)
    for t in ts:
        t.join(timeout=30)
        assert not t.is_alive()
    t0 = time.time()
    while st.loads_pending() and time.time() - t0 < 10:
        time.sleep(0.01)
    assert not errors and st.loads_pending() == 0
    st.close()


@pytest.mark.parametrize("disk", [False, True])
def test_block_store_random_operations_keep_the_contract(tmp_path, disk):
    """Random saves of branching conversations, snapshots, look-ups, reads, thinning and budget pressure: whatever the
    store still returns is byte for byte what was saved under that key, look-ups return a chain of the prompt's own
    blocks with the depth of a real snapshot, and the budgets hold."""
    import random
    rnd = random.Random(5 + disk)
    ram = 48 << 10
    st = H.BlockStore(3, 1, ram_budget=ram, disk_dir=str(tmp_path) if disk else None, disk_budget=(256 << 10) if disk else 0)
    saved, snaps = {}, {}                    # key -> payload; key -> snapshot payload
    convs = []                               # token lists (multiples of 256)
    for step in range(400):
        op = rnd.random()
        if op < 0.45 or not convs:
            base = list(rnd.choice(convs)) if convs and rnd.random() < 0.6 else []
            base = base[:256 * rnd.randrange(0, len(base) // 256 + 1)]
            toks = base + [rnd.randrange(50) for _ in range(256 * rnd.randrange(1, 4))]
            path, _ = st.lookup(toks + [1])
            parent = path[-1] if path else st.root
            for bi in range(len(path), len(toks) // 256):
                h = hash((parent, tuple(toks[bi * 256:(bi + 1) * 256]))) & 0xFFFFFF          # a block's payload is a function of what it holds
                payload = bytes([h % 256]) * (500 + h % 2500)
                k = st.save_block(parent, bi * 256, toks[bi * 256:(bi + 1) * 256], payload)
                if k == 0:
                    break
                assert k == H.BlockStore.key(parent, toks[bi * 256:(bi + 1) * 256])
                saved[k] = payload
                parent = k
                if rnd.random() < 0.5:
                    sp = bytes([(h >> 8) % 256]) * 200
                    if st.save_snapshot(k, sp, None, anchor=rnd.random() < 0.1):
                        snaps[k] = sp
            convs.append(toks)
        elif op < 0.8:
            toks = list(rnd.choice(convs))
            cut = rnd.randrange(1, len(toks) + 1)
            q = toks[:cut] + ([rnd.randrange(50, 60)] * rnd.randrange(0, 300))
            path, depth = st.lookup(q)
            assert len(path) <= len(q) // 256 and 0 <= depth <= len(path)
            parent = st.root
            for bi, k in enumerate(path):                          # a chain of the prompt's own blocks
                assert k == H.BlockStore.key(parent, q[bi * 256:(bi + 1) * 256])
                parent = k
            for k in path:
                got = st.get(k)
                assert got is None or got == saved[k]
            if depth:
                got = st.get(path[depth - 1], snapshot=True)
                assert got is None or got[0] == snaps[path[depth - 1]]
        elif op < 0.9:
            st.thin(rnd.choice([300, 600, 2000]))
        else:
            if disk:
                st.flush()
            s_ = st.stats()
            assert s_["ram_bytes"] <= ram + 4096 or disk          # without a disk tier the RAM budget is enforced at once
    if disk:
        st.flush()
        s_ = st.stats()
        assert s_["disk_bytes"] <= (256 << 10) + 8192
    st.close()


def test_chunker_edit_locality_and_bounds():
    """An edit in the middle of a prompt changes the chunks around it and leaves the rest alone; chunk lengths stay inside
    the minimum / maximum except at a message boundary and at the end."""
    rng = np.random.default_rng(21)
    toks = rng.integers(0, 50000, size=20000).tolist()
    a = H.chunk_prompt(toks, -1)
    edited = list(toks)
    edited[10000:10010] = rng.integers(0, 50000, size=10).tolist()
    b = H.chunk_prompt(edited, -1)
    ha, hb = [c[2] for c in a], [c[2] for c in b]
    assert len(set(ha) ^ set(hb)) <= 6                        # only the chunks next to the edit differ
    before = [c for c in a if c[0] + c[1] <= 9000]
    after = [c for c in a if c[0] >= 13000]
    assert before and after and all(c in b for c in before) and all(c in b for c in after)
    assert all(128 <= c[1] <= 2048 for c in a[:-1]) and 0 < a[-1][1] <= 2048
    assert H.chunk_prompt([], -1) == [] and sum(c[1] for c in H.chunk_prompt(toks[:100], -1)) == 100
