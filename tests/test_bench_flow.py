"""The benchmark script's control flow on CPU, with the engine, the session and the CUDA timing calls replaced by fakes:
the JSON line carries every key of the contract, a failure in an extra run (long prefill, speculative decoding) leaves the
headline in place and is recorded, and a failing token-major prefill falls back to the row-batched path."""
import importlib.util
import json
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeEvent:
    clock = 0.0

    def __init__(self, enable_timing=False):
        self.t = None

    def record(self):
        FakeEvent.clock += 50.0
        self.t = FakeEvent.clock

    def elapsed_time(self, other):
        return other.t - self.t


class FakeDM:
    def __init__(self):
        self.buf = {"amax_idx": torch.tensor([5, 6, 7], dtype=torch.int32)}
        self.rows_host = torch.zeros(128, dtype=torch.int32)
        self.err_word = torch.zeros(4, dtype=torch.int32)
        self.lib = types.SimpleNamespace(qwrt_last_launches=lambda: 321)
        self.error = None

    def weight_bytes(self):
        return 9.8e9

    def check_error(self):
        if self.error:
            msg, self.error = self.error, None
            raise RuntimeError(msg)


class FakeEngine:
    fail_token_major = False

    def __init__(self, opts):
        self.opts = opts
        self.dm = FakeDM()
        self.merge_argmax = None
        self.tp_channels = None
        self.prefiller = types.SimpleNamespace(T=4096, lanes=1)
        self.last_prefill_row = 1
        self.mtp = True
        self.calls = []

    def prefill(self, slot, toks, want_logits=True):
        self.calls.append(("prefill", slot, len(toks), bool(self.opts.prefill_chunk)))
        if FakeEngine.fail_token_major and self.opts.prefill_chunk:
            raise RuntimeError("device error word: code 1 (a bounded wait ran out)")

    def reset(self, slot):
        self.calls.append(("reset", slot))

    def decode_chain(self, slot, tok, n):
        return [(tok + i + 1) % 1000 for i in range(n)]

    def decode(self, slots, toks):
        return [(t + 1) % 1000 for t in toks]


class FakeSession:
    fail_after = None

    def __init__(self, eng, host_cache_bytes=0):
        self.sampler = types.SimpleNamespace(reset_slot=lambda s: None)
        self.n = 0

    def generate(self, reqs, k, force_accept=None):
        self.n += 1
        if FakeSession.fail_after is not None and self.n > FakeSession.fail_after:
            raise RuntimeError("device error word: code 1 detail 553649293")
        return [types.SimpleNamespace(tokens=[r.pending + 1] * (1 + force_accept)) for r in reqs]


class FakeSampler:
    def __init__(self, idx):
        pass

    def start(self):
        pass

    def stop(self):
        pass

    def summary(self):
        return {"sm_mhz": 1900, "sm_max_mhz": 1965, "reasons": []}


@pytest.fixture
def bench(monkeypatch):
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    import qwb200.engine.engine as E
    import qwb200.session.session as S
    import qwb200.utils.clocks as CK
    monkeypatch.setattr(torch.cuda, "set_device", lambda d: None)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a: None)
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    real_tensor = torch.tensor
    monkeypatch.setattr(torch, "tensor", lambda data, device=None, **kw: real_tensor(data, **kw))      # "cuda:0" tensors live on the CPU here
    monkeypatch.setattr(E.Engine, "synthetic", staticmethod(lambda cfg, opts, **kw: FakeEngine(opts)))
    monkeypatch.setattr(S, "Session", FakeSession)
    monkeypatch.setattr(CK, "ClockSampler", FakeSampler)
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    FakeEngine.fail_token_major = False
    FakeSession.fail_after = None
    return mod


def run(bench, monkeypatch, capsys, *argv):
    monkeypatch.setattr(sys, "argv", ["bench.py", "--model", "tiny", "--context", "512", "--prefill-long", "1024", "--mtp-context", "512",
                                      "--steps", "4", "--warmup", "3", "--mtp-steps", "3", *argv])
    left = []
    monkeypatch.setattr(os, "_exit", lambda code: left.append(code))
    rc = bench.main()
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0]), rc, left


def test_the_json_line_carries_the_contract(bench, monkeypatch, capsys):
    out, rc, left = run(bench, monkeypatch, capsys)
    assert rc == 0 and not left, out.get("extras_failed")
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
              "data", "config", "clocks", "e2e", "gpu_launches", "impl"):
        assert k in out, k
    assert out["steps"] == 4 and out["warmup"] == 3 and out["n_gpus"] == 1 and out["impl"] == "ours"
    assert out["value"] == round(4 / 0.05, 2) and out["ms_per_step"] == 12.5            # the fake clock: 50 ms between two records
    assert out["gpu_launches"] == 321 * 4
    assert set(out["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} and out["e2e"]["h2d_bytes_per_step"] == 512
    assert out["prefill"]["path"] == "token-major" and out["prefill_long"]["tokens"] == 1024
    assert [p["accepted"] for p in out["mtp"]["streams_1"]] == [0, 1, 2, 3, 4, 5]
    assert [p["accepted"] for p in out["mtp"]["streams_4"]] == [0, 1, 2, 3, 4, 5]
    assert out["mtp"]["streams_4"][5]["tok_s"] == round(4 * 6 * 3 / 0.05, 1)
    assert "extras_failed" not in out and "not the named model" in out["config"]["model"]


def test_a_failing_extra_leaves_the_headline(bench, monkeypatch, capsys):
    FakeSession.fail_after = 10
    out, rc, left = run(bench, monkeypatch, capsys)
    assert out["value"] == round(4 / 0.05, 2) and out["prefill_long"] is not None
    assert out["mtp"] is None and "mtp" in out["extras_failed"] and "RuntimeError" in out["extras_failed"]["mtp"]
    assert left == [0]                     # the ranks may be out of step: the process leaves without the collective tear-down


def test_token_major_prefill_falls_back(bench, monkeypatch, capsys):
    FakeEngine.fail_token_major = True
    out, rc, left = run(bench, monkeypatch, capsys)
    assert out["prefill"]["path"] == "row-batched" and "token-major prefill failed" in out["prefill"]["note"]
    assert out["prefill_long"] is None and out["value"] > 0 and out["mtp"] is not None


def _rank_main(rank, world, port, fail_rank, q):
    """One rank of a two-rank run on gloo: the same fakes, rank `fail_rank`'s speculative step fails part-way."""
    import contextlib
    import io
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK="0")
    import qwb200.parallel.dist_engine as DE
    import qwb200.session.session as S
    import qwb200.utils.clocks as CK
    torch.cuda.set_device = lambda d: None
    torch.cuda.synchronize = lambda *a: None
    torch.cuda.Event = FakeEvent
    real_tensor, real_device = torch.tensor, torch.device
    torch.tensor = lambda data, device=None, **kw: real_tensor(data, **kw)
    real_init = dist.init_process_group
    dist.init_process_group = lambda backend, device_id=None, **kw: real_init("gloo", rank=rank, world_size=world)
    def make_engine(cfg, opts, world, rank, dev, **kw):
        e = FakeEngine(opts)
        e.tp_channels = [object()]            # the token-major path is on
        return e
    DE.make_engine = make_engine
    S.Session = FakeSession
    CK.ClockSampler = FakeSampler
    FakeSession.fail_after = 10 if rank == fail_rank else None
    FakeEngine.fail_token_major = rank == fail_rank - 100          # 101: rank 1's token-major prefill fails instead
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.argv = ["bench.py", "--gpus", str(world), "--model", "tiny", "--context", "512", "--prefill-long", "1024", "--mtp-context", "512",
                "--steps", "4", "--warmup", "3", "--mtp-steps", "3"]
    left = []
    os_exit, os._exit = os._exit, lambda code: left.append(code)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        mod.main()
    os._exit = os_exit
    q.put((rank, buf.getvalue(), left))


@pytest.mark.parametrize("fail_rank", [-1, 1, 101])
def test_two_ranks_stay_in_step(fail_rank):
    """Two gloo ranks: without a failure rank 0 prints the line and both tear down; when only rank 1's speculative step
    fails, both ranks record the failure at the same sync point, rank 0 still prints the headline and nobody hangs."""
    import multiprocessing as mp
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank_main, args=(r, 2, port, fail_rank, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = {}
    for _ in ps:
        r, text, left = q.get(timeout=120)
        got[r] = (text, left)
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    lines = [ln for ln in got[0][0].splitlines() if ln.startswith("{")]
    assert len(lines) == 1 and not [ln for ln in got[1][0].splitlines() if ln.startswith("{")]
    out = json.loads(lines[0])
    assert out["n_gpus"] == 2 and out["value"] == round(4 / 0.05, 2)
    if fail_rank == 101:
        # only rank 1's token-major prefill failed: both ranks filled the context by the row-batched path and went on together
        assert out["prefill"]["path"] == "row-batched" and "failed" in out["prefill"]["note"] and out["prefill_long"] is None
        assert len(out["mtp"]["streams_1"]) == 6 and "extras_failed" not in out
        return
    assert out["prefill_long"] is not None
    if fail_rank < 0:
        assert "extras_failed" not in out and len(out["mtp"]["streams_4"]) == 6 and got[0][1] == [] and got[1][1] == []
    else:
        assert out["mtp"] is None and "mtp" in out["extras_failed"]
        assert got[0][1] == [0] and got[1][1] == [0]
