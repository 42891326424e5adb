"""Failure detection without a GPU: the collectives' protocol on CPU ranks (late rank, skipped push, dead rank) and
the host heartbeat across processes over a TCP store."""
import multiprocessing as mp
import time

import numpy as np
import pytest


def test_protocol_sums_are_bit_identical_and_late_rank_is_fine():
    from qwb200.parallel.cpu_protocol import CpuWorld, run_ranks
    R, n = 4, 37
    w = CpuWorld(R, 64)
    rng = np.random.default_rng(0)
    vals = rng.standard_normal((3, R, n)).astype(np.float32)

    def body(rk):
        outs = []
        for step in range(3):
            rk.bump()
            if rk.rank == 2 and step == 1:
                time.sleep(0.15)                  # a late rank inside the limit
            rk.put_all(1, vals[step, rk.rank])
            a = rk.reduce(1, n)
            rk.put_cols(2, np.tile(vals[step, rk.rank, :8], R))
            b = rk.reduce(2, 8)
            outs.append((a, b))
        return outs
    res = run_ranks(w, body, spin_seconds=2.0)
    assert all(e.code == 0 for e in w.err)
    for step in range(3):
        want = np.zeros(n, np.float32)
        for r in range(R):
            want += vals[step, r]                 # rank order: what every rank must have computed
        for r in range(R):
            assert np.array_equal(res[r][step][0], want)
            assert np.array_equal(res[r][step][1], res[0][step][1])


def test_skipped_push_times_out_with_the_culprit_and_stops_all_waits():
    from qwb200.parallel.cpu_protocol import ERR_WAIT_TIMEOUT, CpuWorld, run_ranks
    R = 3
    w = CpuWorld(R, 16)

    def body(rk):
        rk.bump()
        if rk.rank != 1:                          # rank 1 "forgets" collective 5
            rk.put_all(5, np.ones(4, np.float32))
        a = rk.reduce(5, 4)
        t0 = time.monotonic()
        b = rk.reduce(6, 4)                       # nobody pushed 6: must return at once because the error word is set
        return a, b, time.monotonic() - t0
    t0 = time.monotonic()
    res = run_ranks(w, body, spin_seconds=0.3)
    assert time.monotonic() - t0 < 3.0
    for r in range(R):
        a, b, dt = res[r]
        assert a is None and b is None and dt < 0.1
        assert w.err[r].code == ERR_WAIT_TIMEOUT
        assert (w.err[r].detail >> 24) & 0x3F == 1 and w.err[r].detail & 0xFFFFFF == 5      # waiting for rank 1, collective 5


def test_dead_rank_is_noticed_by_its_peers():
    from qwb200.parallel.cpu_protocol import CpuWorld, run_ranks
    w = CpuWorld(2, 8)

    def body(rk):
        rk.bump()
        if rk.rank == 0:
            raise RuntimeError("rank 0 died before its push")
        rk.put_all(1, np.ones(2, np.float32))
        return rk.reduce(1, 2)
    res = run_ranks(w, body, spin_seconds=0.2)
    assert isinstance(res[0], RuntimeError) and res[1] is None and w.err[1].code != 0 and (w.err[1].detail >> 24) & 0x3F == 0


def _hb_worker(rank, world, port, q):
    from torch.distributed import TCPStore
    from qwb200.parallel.heartbeat import Heartbeat
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, interval=0.05, limit=3.0)      # generous: a starved process on a busy box is not a failure
    hb.start()
    store.set(f"ready/{rank}", "1")
    for r in range(world):
        store.wait([f"ready/{r}"])
    steps = 0
    try:
        for step in range(200):
            hb.check()                            # before every launch
            steps += 1
            if rank == 2 and step == 3:
                hb.leave("shutting down")         # between steps, nothing in flight
                q.put((rank, steps, "left"))
                time.sleep(1.0)                   # keep the store's clients alive while the others notice
                store.set(f"done/{rank}", "1")
                return
            if rank == 1 and step == 3:
                hb.stop_flag.set()                # rank 1 stops beating without saying anything
                time.sleep(5.0)
                q.put((rank, steps, "silent"))
                store.set(f"done/{rank}", "1")
                return
            time.sleep(0.05)
        q.put((rank, steps, "never noticed"))
    except RuntimeError as ex:
        q.put((rank, steps, str(ex)))
        if rank == 0:                             # the store's server outlives its clients: wait until they say they are done
            try:
                store.wait([f"done/{r}" for r in range(1, world)], __import__("datetime").timedelta(seconds=30))
            except Exception:
                pass
            time.sleep(0.3)
        else:
            store.set(f"done/{rank}", "1")


def test_heartbeat_across_processes():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket
    with socket.socket() as sk:                    # a port nobody holds right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ps = [ctx.Process(target=_hb_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in ps:
        p.start()
    got = {}
    for _ in range(3):
        r, steps, msg = q.get(timeout=60)
        got[r] = (steps, msg)
    for p in ps:
        p.join(timeout=30)
    assert got[2] == (4, "left")
    assert "peer failure" in got[0][1] and ("rank 2: shutting down" in got[0][1] or "rank 1: silent" in got[0][1])
    assert 1 <= got[0][0] < 60                     # noticed within a few steps, long before the loop's end


# ---- the prefill channel's protocol (flags, tickets, per-kind sequence numbers) on CPU ranks
def test_tp_channel_sums_in_rank_order_and_counts_per_kind():
    import numpy as np
    from qwb200.parallel.cpu_protocol import TpWorld, run_tp_ranks
    w = TpWorld(4, kinds=3, words=64)

    def body(rk):
        outs = []
        for step in range(5):                             # kinds interleaved: each keeps its own count
            for kind in (0, 2):
                v = np.arange(48, dtype=np.float32) * (rk.rank + 1) + step + kind
                seq = rk.send(kind, v, ctas=5)
                got = rk.receive(kind, 48, seq)
                outs.append(got)
                rk.rendezvous()                           # the buffer of a kind is reused: everybody has read it
        return outs, list(rk.seq)
    res = run_tp_ranks(w, body, spin_seconds=5.0)
    assert all(e.code == 0 for e in w.err)
    for outs, seqs in res:
        assert seqs == [5, 0, 5]
        i = 0
        for step in range(5):
            for kind in (0, 2):
                want = sum(np.arange(48, dtype=np.float32) * (r + 1) + step + kind for r in range(4))
                assert np.array_equal(outs[i], want)
                i += 1


def test_tp_channel_late_host_times_out_without_a_rendezvous_and_not_with_one():
    """A rank whose host reaches the chunk later than its peers' bounded wait: without a rendezvous before the chunk the
    peers give up and name it; with one (or with a limit longer than the delay) the chunk completes."""
    import time
    import numpy as np
    from qwb200.parallel.cpu_protocol import ERR_WAIT_TIMEOUT, TpWorld, run_tp_ranks

    def chunk(rk, rendezvous, delay):
        if rk.rank == 1:
            time.sleep(delay)                             # its host is still allocating buffers
        if rendezvous and not rk.rendezvous():
            return None
        seq = rk.send(0, np.full(8, rk.rank + 1.0, dtype=np.float32))
        return rk.receive(0, 8, seq)
    w = TpWorld(2, kinds=1, words=8)
    res = run_tp_ranks(w, lambda rk: chunk(rk, False, 0.6), spin_seconds=0.2)
    assert res[0] is None and w.err[0].code == ERR_WAIT_TIMEOUT
    assert (w.err[0].detail >> 24) & 7 == 1 and w.err[0].detail & 0xffffff == 1          # waited for rank 1, collective 1
    w = TpWorld(2, kinds=1, words=8)
    res = run_tp_ranks(w, lambda rk: chunk(rk, True, 0.6), spin_seconds=0.2)
    assert all(e.code == 0 for e in w.err) and np.array_equal(res[0], np.full(8, 3.0)) and np.array_equal(res[1], res[0])
    w = TpWorld(2, kinds=1, words=8)
    res = run_tp_ranks(w, lambda rk: chunk(rk, False, 0.3), spin_seconds=5.0)               # a limit above the delay
    assert all(e.code == 0 for e in w.err) and np.array_equal(res[0], np.full(8, 3.0))


def test_tp_channel_missing_rank_is_reported_once_and_everyone_stops_waiting():
    import numpy as np
    from qwb200.parallel.cpu_protocol import ERR_WAIT_TIMEOUT, TpWorld, run_tp_ranks
    w = TpWorld(4, kinds=2, words=16)

    def body(rk):
        if rk.rank == 2:
            return "left"                                 # never sends
        seq = rk.send(1, np.ones(16, dtype=np.float32))
        first = rk.receive(1, 16, seq)
        t0 = time.monotonic()
        seq2 = rk.send(0, np.ones(4, dtype=np.float32))
        second = rk.receive(0, 4, seq2)                   # the error word is set: no second wait of the full limit
        return first, second, time.monotonic() - t0
    import time
    res = run_tp_ranks(w, body, spin_seconds=0.3)
    for r in (0, 1, 3):
        first, second, dt = res[r]
        assert first is None and second is None and dt < 0.2
        assert w.err[r].code == ERR_WAIT_TIMEOUT and (w.err[r].detail >> 24) & 7 == 2
