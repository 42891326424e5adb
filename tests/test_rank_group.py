"""The command channel of a multi-GPU engine (``parallel/rank_group.py``) with recorder workers instead of engines:
calls reach every rank in order, and a rank that raises, dies or hangs is detected and named.  No GPU involved: the
failures are made on the host (a worker that raises, exits, or sleeps)."""
import ast
import os
import time

import pytest


class Local:
    def __init__(self):
        self.log = []

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)

        def method(*args):
            self.log.append((name, args))
            if name == "refuse":
                raise ValueError("no room")
            return len(self.log)
        return method


def start(world=3, **inject):
    from qwb200.parallel.rank_group import RankGroup
    loc = Local()
    g = RankGroup.spawn(world, ["--fake"], dict(inject), lambda: loc, ready_timeout=60, ack_timeout=inject.pop("ack_timeout", 20))
    return g, loc


def test_calls_reach_every_rank_in_order(tmp_path):
    g, loc = start(3)
    try:
        assert g.call("acquire", [1, 2, 3], 16) == 1
        assert g.decode([0], [5]) == 2                      # attribute form
        with pytest.raises(ValueError):                     # a refusal raised on rank 0 is the caller's error, not a failure
            g.call("refuse", 1)
        assert g.failure() == ""
        g.call("dump", str(tmp_path / "log"))
        want = [("acquire", ([1, 2, 3], 16)), ("decode", ([0], [5])), ("refuse", (1,))]
        assert loc.log[:3] == want
        for r in (1, 2):
            got = ast.literal_eval(open(str(tmp_path / "log") + f".rank{r}").read())
            assert got[:3] == want
    finally:
        g.shutdown()
    assert all(p.poll() == 0 for p in g.procs)


def test_a_rank_that_raises_alone_fails_the_group():
    from qwb200.parallel.rank_group import RankFailure
    g, loc = start(3, fail_on="generate", victim=2)
    try:
        g.call("prefill_some", 0, 128)
        with pytest.raises(RankFailure) as e:
            g.call("generate", [(0, 7, 4)], 3)
        assert "rank 2 failed in 'generate'" in str(e.value) and "injected failure" in str(e.value)
        assert "rank 2" in g.failure()
        with pytest.raises(RankFailure):                    # sticky: nothing runs any more
            g.call("decode", [0], [1])
        assert [n for n, _ in loc.log] == ["prefill_some", "generate"]
    finally:
        g.shutdown()


def test_a_rank_that_exits_is_noticed():
    from qwb200.parallel.rank_group import RankFailure
    g, loc = start(2, exit_on="decode", victim=1)
    try:
        with pytest.raises(RankFailure) as e:
            g.call("decode", [0], [1])
        assert "rank 1 is gone" in str(e.value)
        time.sleep(0.2)
        assert "rank 1" in g.failure()
    finally:
        g.shutdown()


def test_a_rank_that_hangs_times_out():
    from qwb200.parallel.rank_group import RankFailure
    g, loc = start(2, hang_on="generate", victim=1, ack_timeout=1.0)
    try:
        t0 = time.time()
        with pytest.raises(RankFailure) as e:
            g.call("generate", [], 0)
        assert "rank 1 did not answer 'generate'" in str(e.value) and time.time() - t0 < 10
    finally:
        g.shutdown(timeout=1.0)
