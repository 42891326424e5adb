"""Lock-step guard on two gloo ranks (CPU): a rank that fails between two sync points skips its work, both ranks raise at
the sync point, nobody hangs, and without a failure the guard is a plain barrier."""
import multiprocessing as mp
import os

import pytest


def worker(rank, world, port, fail_rank, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from qwb200.utils.lockstep import Lockstep
    g = Lockstep(dist, torch.device("cpu"))
    done = []
    g.sync_point()                                         # nobody failed: a barrier
    done.append("a")

    def work():
        if rank == fail_rank:
            raise ValueError("boom on this rank only")
        done.append("b")
        return 7
    r1 = g.attempt(work, default=-1)
    r2 = g.attempt(lambda: done.append("c") or 8, default=-2)      # after a failure the rank's work is skipped
    try:
        g.sync_point()
        outcome = "passed"
    except RuntimeError as ex:
        outcome = str(ex)
    q.put((rank, done, r1, r2, outcome))
    dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [1, -1])
def test_failure_on_one_rank_raises_on_both_at_the_sync_point(fail_rank):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket
    with socket.socket() as sk:                    # a port nobody holds right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ps = [ctx.Process(target=worker, args=(r, 2, port, fail_rank, q)) for r in range(2)]
    [p.start() for p in ps]
    got = sorted(q.get(timeout=120) for _ in ps)
    [p.join(30) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    (r0, done0, a0, b0, out0), (r1, done1, a1, b1, out1) = got
    if fail_rank < 0:
        assert out0 == out1 == "passed" and done0 == done1 == ["a", "b", "c"] and (a0, b0) == (7, 8)
        return
    assert done0 == ["a", "b", "c"] and (a0, b0) == (7, 8)              # the healthy rank did its work ...
    assert done1 == ["a"] and (a1, b1) == (-1, -2)                      # ... the failed one skipped the rest of its own
    assert out0 == "failed on another rank" and "boom" in out1          # ... and both raised together


def test_single_rank_guard_checks_the_device():
    from qwb200.utils.lockstep import Lockstep
    calls = []

    def check():
        calls.append(1)
        raise RuntimeError("device error word: code 1")
    g = Lockstep(None, None, check=check, sync=lambda: calls.append(0))
    with pytest.raises(RuntimeError, match="device error word"):
        g.sync_point()
    assert g.attempt(lambda: 5, default=9) == 9 and calls[0] == 0
