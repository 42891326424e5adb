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
