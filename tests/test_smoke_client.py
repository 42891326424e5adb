"""The deployment smoke client against the HTTP app on a fake engine: all checks pass on a healthy server, and the
report names the failing check when the engine has failed."""
import asyncio

import pytest

aiohttp = pytest.importorskip("aiohttp")
pytest.importorskip("tokenizers")
from aiohttp.test_utils import TestClient, TestServer  # noqa: E402

from server_fixtures import make_server  # noqa: E402


def run_smoke(srv, **kw):
    from qwserve.api import make_app
    from qwserve.smoke import run_checks

    async def go():
        async with TestClient(TestServer(make_app(srv))) as c:
            base = str(c.make_url("")).rstrip("/")
            return await run_checks(c.session, base, **kw)
    return asyncio.run(go())


def test_smoke_passes_on_a_healthy_server_with_follow_up():
    srv, sched, eng, pr = make_server("sure</think>Hello there.")
    rep = run_smoke(srv, max_tokens=32, follow_up=True)
    sched.shutdown()
    assert rep["ok"], rep
    assert [c["name"] for c in rep["checks"]] == ["health", "models", "tokenize", "chat", "chat_stream", "follow_up"]
    assert all(c["ok"] for c in rep["checks"])
    assert rep["checks"][3]["completion_tokens"] >= 1 and rep["checks"][4]["frames"] >= 1


def test_smoke_names_the_failing_check():
    srv, sched, eng, pr = make_server("x</think>y")
    eng.failed_with = "rank 1 stopped answering"
    rep = run_smoke(srv)
    sched.shutdown()
    assert not rep["ok"]
    assert rep["checks"][-1]["ok"] is False and rep["checks"][-1]["name"] in ("health", "chat")


def test_idle_wait_needs_a_quiet_spell_without_completions():
    """Idle = nothing in flight and no request finished for the whole spell; a request in flight or one that completed
    in between restarts the spell; an unreachable server is never idle."""
    from qwserve.idle import wait_idle
    t = [0.0]
    clock, sleep = (lambda: t[0]), (lambda s: t.__setitem__(0, t[0] + s))
    seq = iter([(1, 0), (0, 1), (0, 1), (0, 2), (0, 2), (0, 2), (0, 2), (0, 2)])          # (busy, completed) per poll, 5 s apart
    assert wait_idle("x", 12, 5, 100, probe=lambda u: next(seq), clock=clock, sleep=sleep)
    assert t[0] == 35.0          # a completion is seen at t=15, the quiet spell starts at the next poll (t=20) and is 12 s old at t=35
    t[0] = 0.0
    assert not wait_idle("x", 12, 5, 40, probe=lambda u: (1, 0), clock=clock, sleep=sleep)

    def down(u):
        raise OSError("connection refused")
    t[0] = 0.0
    assert not wait_idle("x", 5, 5, 30, probe=down, clock=clock, sleep=sleep)


def test_idle_probe_reads_the_health_endpoint():
    from qwserve.api import make_app
    from qwserve.idle import busy_and_done
    srv, sched, eng, pr = make_server("a</think>b")

    async def go():
        async with TestClient(TestServer(make_app(srv))) as c:
            base = str(c.make_url("")).rstrip("/")
            loop = asyncio.get_running_loop()
            before = await loop.run_in_executor(None, busy_and_done, base)
            await (await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})).json()
            after = await loop.run_in_executor(None, busy_and_done, base)
            return before, after
    before, after = asyncio.run(go())
    sched.shutdown()
    assert before == (0, 0) and after == (0, 1)
