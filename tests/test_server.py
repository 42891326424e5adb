"""HTTP + scheduler tier on a fake engine: API shapes, streaming == non-streaming, reasoning / tool routing,
thinking budget, stop strings, admission without head-of-line blocking, failure isolation, health, dashboard
(the reference's server tests cover the same ground: server/tests/test_api.py, test_admission.py,
test_isolation.py, test_health.py, test_thinking.py, test_concurrency.py)."""
import asyncio
import json
import threading
import time

import pytest

from server_fixtures import make_prompter, make_server

aiohttp = pytest.importorskip("aiohttp")
from aiohttp.test_utils import TestClient, TestServer  # noqa: E402


def with_client(srv, fn):
    from qwserve.api import make_app

    async def go():
        async with TestClient(TestServer(make_app(srv))) as c:
            return await fn(c)
    return asyncio.run(go())


async def sse(resp):
    frames = []
    async for line in resp.content:
        line = line.decode().strip()
        if line.startswith("data: ") and line != "data: [DONE]":
            frames.append(json.loads(line[6:]))
    return frames


MSG = [{"role": "user", "content": "hi"}]


def test_chat_plain_and_usage():
    srv, sched, eng, pr = make_server("thinking hard</think>The answer is 4.")

    async def fn(c):
        r = await c.post("/v1/chat/completions", json={"messages": MSG, "logprobs": True, "top_logprobs": 2})
        assert r.status == 200
        return await r.json()
    out = with_client(srv, fn)
    ch = out["choices"][0]
    assert ch["message"]["content"] == "The answer is 4."
    assert ch["message"]["reasoning_content"] == "thinking hard"
    assert ch["finish_reason"] == "stop"
    u = out["usage"]
    assert u["prompt_tokens"] == len(pr.encode(pr.render(MSG)))
    assert u["completion_tokens_details"]["reasoning_tokens"] == len("thinking hard")
    lp = ch["logprobs"]["content"]
    assert len(lp) == len("thinking hard") + len("The answer is 4.") and len(lp[0]["top_logprobs"]) == 2
    assert out["timings"]["predicted_n"] == u["completion_tokens"]
    sched.shutdown()


def test_stream_equals_nonstream_and_utf8():
    text = "plan</think>naïve café 日本語 ok"
    srv, sched, eng, pr = make_server(text)

    async def fn(c):
        a = await (await c.post("/v1/chat/completions", json={"messages": MSG})).json()
        r = await c.post("/v1/chat/completions", json={"messages": MSG, "stream": True, "stream_options": {"include_usage": True}})
        return a, await sse(r)
    a, frames = with_client(srv, fn)
    content = "".join(f["choices"][0]["delta"].get("content") or "" for f in frames if f["choices"])
    reasoning = "".join(f["choices"][0]["delta"].get("reasoning_content") or "" for f in frames if f["choices"])
    assert content == a["choices"][0]["message"]["content"] == "naïve café 日本語 ok"
    assert reasoning == "plan"
    assert "�" not in content
    assert frames[-1]["usage"]["completion_tokens"] == a["usage"]["completion_tokens"]
    assert [f for f in frames if f["choices"]][-1]["choices"][0]["finish_reason"] == "stop"
    sched.shutdown()


def test_thinking_disabled_and_budget():
    from qwserve.prompt import resolve_thinking
    assert resolve_thinking({"chat_template_kwargs": {"enable_thinking": False}})[0] is False
    assert resolve_thinking({"reasoning_effort": "none"})[0] is False
    assert resolve_thinking({"reasoning_effort": "low"}) == (True, "low", 1024)
    assert resolve_thinking({"thinking": {"type": "enabled", "budget_tokens": 77}}) == (True, None, 77)
    assert resolve_thinking({"thinking": {"type": "disabled"}})[0] is False
    assert resolve_thinking({"thinking_budget": 5}, None, 100)[2] == 5
    # a model that never stops thinking is closed by force after the budget
    srv, sched, eng, pr = make_server("x" * 500)

    async def fn(c):
        return await (await c.post("/v1/chat/completions", json={"messages": MSG, "thinking_budget": 10, "max_tokens": 40})).json()
    out = with_client(srv, fn)
    m = out["choices"][0]["message"]
    assert m["reasoning_content"].startswith("x" * 10) and len(m["reasoning_content"].strip()) == 10
    assert m["content"].startswith("\n\n") and set(m["content"].strip()) == {"x"}
    assert out["choices"][0]["finish_reason"] == "length"
    assert sched.stats["forced_think_close"] == 1
    sched.shutdown()


def test_tool_call_routing():
    reply = "</think>Let me look.<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>"
    srv, sched, eng, pr = make_server(reply)
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
        "city": {"type": "string"}, "days": {"type": "integer"}}}}}]

    async def fn(c):
        a = await (await c.post("/v1/chat/completions", json={"messages": MSG, "tools": tools})).json()
        r = await c.post("/v1/chat/completions", json={"messages": MSG, "tools": tools, "stream": True})
        return a, await sse(r)
    a, frames = with_client(srv, fn)
    ch = a["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["content"] == "Let me look."
    call = ch["message"]["tool_calls"][0]
    assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Paris", "days": 3}
    streamed = [f["choices"][0]["delta"]["tool_calls"][0] for f in frames if f["choices"] and "tool_calls" in f["choices"][0]["delta"]]
    assert len(streamed) == 1 and streamed[0]["function"]["name"] == "get_weather" and streamed[0]["index"] == 0
    sched.shutdown()


def test_stop_string_and_completions_and_tokenize():
    srv, sched, eng, pr = make_server("one two STOP three")

    async def fn(c):
        a = await (await c.post("/v1/completions", json={"prompt": "abc", "stop": ["STOP"]})).json()
        r = await c.post("/v1/completions", json={"prompt": "abc", "stop": "STOP", "stream": True})
        frames = await sse(r)
        t = await (await c.post("/tokenize", json={"prompt": "abc"})).json()
        t2 = await (await c.post("/tokenize", json={"messages": MSG})).json()
        m = await (await c.get("/v1/models")).json()
        bad = await c.post("/v1/completions", json={"prompt": {"no": 1}})
        bad2 = await c.post("/v1/chat/completions", json={"messages": MSG, "n": 2})
        return a, frames, t, t2, m, bad.status, bad2.status
    a, frames, t, t2, m, bad, bad2 = with_client(srv, fn)
    assert a["choices"][0]["text"] == "one two " and a["choices"][0]["finish_reason"] == "stop"
    assert "".join(f["choices"][0]["text"] for f in frames) == "one two "
    assert t["count"] == 3 and t["tokens"] == pr.encode("abc") and t2["count"] == len(pr.encode(pr.render(MSG)))
    assert m["data"][0]["id"] == "qw-test" and m["data"][0]["max_model_len"] == 4096
    assert bad == 400 and bad2 == 400
    sched.shutdown()


def test_parallel_equals_serial():
    pr = make_prompter()
    reply = lambda prompt: pr.encode("</think>echo:" + pr.decode(prompt)[-12:])
    srv, sched, eng, _ = make_server(reply=reply, step_seconds=0.001)
    prompts = [f"question number {i}" for i in range(8)]

    async def fn(c):
        async def one(p):
            return (await (await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": p}], "max_tokens": 64})).json())["choices"][0]["message"]["content"]
        serial = [await one(p) for p in prompts]
        par = await asyncio.gather(*[one(p) for p in prompts])
        return serial, list(par)
    serial, par = with_client(srv, fn)
    assert serial == par and len(set(serial)) == 1 or serial == par
    assert "generate" in eng.calls
    sched.shutdown()


def test_admission_skips_request_that_does_not_fit():
    """A request too large for the free slots waits; later, smaller ones are admitted past it."""
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(4096, 256), step_seconds=0.002)
    done = {}

    def mk(name, n_prompt, max_new):
        ev = threading.Event()
        r = Request(tokens=Tokens([65] * n_prompt), max_new=max_new, sampling=Sampling(), stop_ids=[eng.eos],
                    on_done=lambda reason, name=name, ev=ev: (done.__setitem__(name, (reason, time.time())), ev.set()))
        return r, ev
    eng.reply = lambda prompt: [66] * 200
    big1, e1 = mk("big1", 1000, 300)       # takes the 4096 slot
    big2, e2 = mk("big2", 1000, 300)       # needs the 4096 slot too: must wait
    small, e3 = mk("small", 10, 5)         # fits the 256 slot while big2 waits
    for r in (big1, big2, small):
        sched.submit(r)
    assert e3.wait(10) and e1.wait(10) and e2.wait(10)
    assert done["small"][1] < done["big2"][1]
    assert done["big1"][0] == done["big2"][0] == "stop" and done["small"][0] == "length"
    sched.shutdown()


def test_failure_isolation_and_health():
    srv, sched, eng, pr = make_server("</think>fine", step_seconds=0.002)
    eng.poison = pr.encode("Z")[0]

    async def fn(c):
        bad = await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "ZZZ"}]})
        good = await c.post("/v1/chat/completions", json={"messages": MSG})
        h = await c.get("/health")
        return bad.status, await bad.json(), good.status, (await good.json())["choices"][0]["message"]["content"], h.status, await h.json()
    bs, bj, gs, gc, hs, hj = with_client(srv, fn)
    assert bs == 500 and "poisoned" in bj["error"]["message"]
    assert gs == 200 and gc == "fine"
    assert hs == 200 and hj["status"] == "ok" and hj["decode"]["failed"] == 1
    # an engine that reports a failure turns /health into 503
    eng.failed_with = "rank 2: device lost"

    async def fn2(c):
        h = await c.get("/health")
        return h.status, await h.json()
    hs, hj = with_client(srv, fn2)
    assert hs == 503 and "device lost" in hj["reason"]
    sched.shutdown()


def test_generate_error_fails_only_the_culprit():
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(512, 512, 512), step_seconds=0.005)
    eng.reply = lambda prompt: [66] * 30
    res = {}
    evs = []
    reqs = []
    for i in range(3):
        ev = threading.Event()
        evs.append(ev)
        reqs.append(Request(tokens=Tokens([65] * 8), max_new=50, sampling=Sampling(), stop_ids=[eng.eos],
                            on_done=lambda reason, i=i, ev=ev: (res.__setitem__(i, reason), ev.set())))
    for r in reqs:
        sched.submit(r)
    while not all(r.slot >= 0 and r.prefill_done for r in reqs):
        time.sleep(0.002)
    eng.generate_error[reqs[1].slot] = "bad row"
    assert all(ev.wait(10) for ev in evs)
    assert res[1].startswith("error: bad row") and res[0] == "stop" and res[2] == "stop"
    assert sched.health() is None
    sched.shutdown()


def test_failure_after_state_change_is_not_retried():
    """A step that failed after the engine had advanced some slots fails the whole batch: stepping the others again
    would decode their pending tokens twice."""
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(512, 512), step_seconds=0.005)
    eng.reply = lambda prompt: [66] * 30
    res, evs, reqs = {}, [], []
    for i in range(2):
        ev = threading.Event()
        evs.append(ev)
        reqs.append(Request(tokens=Tokens([65] * 8), max_new=50, sampling=Sampling(), stop_ids=[eng.eos],
                            on_done=lambda reason, i=i, ev=ev: (res.__setitem__(i, reason), ev.set())))
    for r in reqs:
        sched.submit(r)
    while not all(r.slot >= 0 and r.prefill_done for r in reqs):
        time.sleep(0.002)
    calls_before = eng.generate_calls if hasattr(eng, "generate_calls") else None
    eng.generate_error[reqs[1].slot] = "step failed after slot state changed: device error"
    assert all(ev.wait(10) for ev in evs)
    assert res[0].startswith("error: step failed after slot state changed") and res[1].startswith("error: step failed")
    sched.shutdown()


def test_hung_engine_call_is_unhealthy():
    srv, sched, eng, pr = make_server("ok", stuck_seconds=0.2)
    eng.generate_block = threading.Event()
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    sched.submit(Request(tokens=Tokens([65] * 4), max_new=8, sampling=Sampling(), stop_ids=[eng.eos]))
    t0 = time.time()
    while sched.health() is None and time.time() - t0 < 5:
        time.sleep(0.05)
    assert "engine call running" in (sched.health() or "")
    eng.generate_block.set()           # let the thread go so the test process can end cleanly
    time.sleep(0.05)
    assert sched.health() is None
    sched.shutdown()


def test_short_prompts_prefill_first_and_single_caller():
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(8192, 8192), piece=512)
    eng.reply = lambda prompt: [66]
    evs = []
    eng.generate_block = None
    long_r = Request(tokens=Tokens([65] * 4000), max_new=2, sampling=Sampling(), stop_ids=[eng.eos])
    short_r = Request(tokens=Tokens([65] * 100), max_new=2, sampling=Sampling(), stop_ids=[eng.eos])
    for r in (long_r, short_r):
        ev = threading.Event()
        evs.append(ev)
        r.on_done = lambda reason, ev=ev: ev.set()
    sched.inbox.put(long_r)
    sched.inbox.put(short_r)
    assert all(ev.wait(10) for ev in evs)
    assert short_r.t_first <= long_r.t_first
    sched.shutdown()


def test_dashboard_and_shutdown_persist():
    srv, sched, eng, pr = make_server("</think>hi")

    async def fn(c):
        await c.post("/v1/chat/completions", json={"messages": MSG})
        page = await c.get("/")
        again = await c.get("/dashboard", headers={"If-None-Match": page.headers["ETag"]})
        bad = await c.get("/metrics.json?tail=lots")
        m = await c.get("/metrics.json?tail=5")
        assert again.status == 304 and bad.status == 400
        return page.status, (await page.text())[:15], await m.json()
    ps, head, m = with_client(srv, fn)
    assert ps == 200 and head.lower().startswith("<!doctype html>")
    assert m["model"] == "qw-test" and m["healthy"] is True and m["counts"]["completed"] == 1
    assert eng.persisted == 1          # leaving the app persists the prefix cache


def test_metrics_rings_and_fake_nvml():
    from qwserve.dashboard.collector import Collector, Gpus
    from qwserve.dashboard.metrics import Metrics
    m = Metrics(seconds=3)
    for i in range(5):
        m.push({"a": i}, now=100.0 + i)
    s = m.snapshot()
    assert s["series"]["a"] == [2.0, 3.0, 4.0] and len(s["t"]) == 3
    assert m.rate("c", 10, 1.0) == 0.0 and m.rate("c", 30, 3.0) == 10.0

    class U:
        gpu = 50
    class M:
        used, total = 2**31, 2**33
    class Nv:
        def nvmlInit(self): pass
        def nvmlDeviceGetCount(self): return 2
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetUtilizationRates(self, h): return U
        def nvmlDeviceGetMemoryInfo(self, h): return M
        def nvmlDeviceGetPowerUsage(self, h): return 700000
        def nvmlDeviceGetTemperature(self, h, k): return 55
        def nvmlDeviceGetClockInfo(self, h, k): return 1900
    g = Gpus(Nv()).sample()
    assert len(g) == 2 and g[1]["power_w"] == 700.0 and g[0]["mem_used_gb"] == 2.0


def test_request_sharing_a_long_prefix_waits_for_the_one_in_flight():
    """Two prompts with the same first 1,024 tokens: the second is not admitted while the first is still prefilling, so it
    finds the shared part in the prefix cache; an unrelated prompt is admitted at once."""
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(8192, 8192, 8192), step_seconds=0.002, start=False)
    shared = [65 + (i % 20) for i in range(1500)]
    a = Request(tokens=Tokens(shared + [70] * 3000), max_new=4, sampling=Sampling(), stop_ids=[eng.eos])
    b = Request(tokens=Tokens(shared + [71] * 10), max_new=4, sampling=Sampling(), stop_ids=[eng.eos])
    c = Request(tokens=Tokens([90] * 1200), max_new=4, sampling=Sampling(), stop_ids=[eng.eos])
    for r in (a, b, c):
        r.in_think = False
        sched.waiting.append(r)
    sched._admit()
    assert a.slot >= 0 and c.slot >= 0 and b.slot < 0 and list(sched.waiting) == [b]
    sched._prefill()                                   # one piece of each: `a` is still not in
    assert not a.prefill_done
    sched._admit()
    assert b.slot < 0
    while sched.prefilling:
        sched._prefill()
    sched._admit()
    assert b.slot >= 0


def test_short_prompts_are_prefilled_by_one_engine_call():
    """Three prompts whose uncached part fits one piece go in with a single prefill_batch call and each gets its first
    token; a long prompt beside them keeps its own pieces; a failing batch call fails exactly its requests."""
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(8192, 8192, 8192, 8192), start=False)
    firsts = {}

    def req(n, tag):
        r = Request(tokens=Tokens([65 + (i % 7) + tag for i in range(n)]), max_new=4, sampling=Sampling(), stop_ids=[eng.eos],
                    on_token=lambda t, lp, top, tag=tag: firsts.setdefault(tag, t))
        r.in_think = False
        return r
    long_, a, b, c = req(5000, 0), req(300, 1), req(700, 2), req(120, 3)
    for r in (long_, a, b, c):
        sched.waiting.append(r)
    sched._admit()
    assert all(r.slot >= 0 for r in (long_, a, b, c))
    sched._prefill()
    assert eng.calls.count("prefill_batch") == 1 and "prefill_some" not in eng.calls
    assert a.prefill_done and b.prefill_done and c.prefill_done and not long_.prefill_done
    assert set(firsts) == {1, 2, 3} and sched.stats["batched_prefills"] == 1
    assert sorted(eng.prefill_order) == sorted([a.slot, b.slot, c.slot])
    while sched.prefilling:
        sched._prefill()                               # the long prompt goes on piece by piece, alone
    assert long_.prefill_done and eng.calls.count("prefill_batch") == 1 and eng.calls.count("prefill_some") == 3
    # a batch call that raises: its requests fail, the scheduler goes on
    srv2, sched2, eng2, _ = make_server("ok", slots=(4096, 4096, 4096), start=False)
    x, y = req(200, 4), req(300, 5)
    for r in (x, y):
        sched2.waiting.append(r)
    sched2._admit()

    def boom(slots, max_tokens):
        raise RuntimeError("engine said no")
    eng2.prefill_batch = boom
    sched2._prefill()
    assert "engine said no" in x.error and "engine said no" in y.error and not sched2.prefilling


def test_watchdog_exits_only_after_the_grace_and_forgets_a_recovery(monkeypatch):
    """The watchdog thread: an engine failure that lasts longer than the grace ends the process with code 3 (so that a
    supervisor restarts it); an unhealthy spell that ends within the grace is forgotten."""
    import os
    from qwserve.scheduler import Scheduler
    from server_fixtures import FakeEngine
    logs, exits = [], []
    eng = FakeEngine(lambda p: [66])
    sched = Scheduler(eng, exit_grace=3.0, log=logs.append)

    def fake_exit(code):
        exits.append(code)
        sched.stop_flag.set()
    monkeypatch.setattr(os, "_exit", fake_exit)

    def wait_for(cond, limit):
        t0 = time.time()
        while not cond() and time.time() - t0 < limit:
            time.sleep(0.05)
        return cond()
    sched.start(watchdog=True)
    eng.failed_with = "rank 2 is gone"
    assert wait_for(lambda: any("unhealthy: engine failure: rank 2 is gone" in ln for ln in logs), 2.5)
    assert not exits                                        # seen, but the grace has not passed
    eng.failed_with = ""
    assert wait_for(lambda: sched.unhealthy_since == 0.0, 2.5) and not exits      # healthy again: the spell is forgotten
    eng.failed_with = "rank 2 is gone"
    t0 = time.time()
    assert wait_for(lambda: bool(exits), 12)
    assert exits == [3] and any(ln.startswith("exiting after") for ln in logs)
    assert time.time() - t0 >= 3.0                          # a full grace counted from the new spell, not from the first one
    sched.shutdown()


def test_request_and_stats_log_lines():
    """One line per finished request with its phases, and a stats line at most every log interval while there is work."""
    import re
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    logs = []
    srv, sched, eng, pr = make_server("ok", log=logs.append, start=False)
    sched.log_interval = 0.05
    sched.start(watchdog=False)
    done = threading.Event()
    r = Request(tokens=Tokens([65] * 300), max_new=8, sampling=Sampling(), stop_ids=[eng.eos], rid="abc123", on_done=lambda reason: done.set())
    sched.submit(r)
    assert done.wait(5)
    t0 = time.time()
    while not any(ln.startswith("stats:") for ln in logs) and time.time() - t0 < 4:
        time.sleep(0.05)
    sched.shutdown()
    req = [ln for ln in logs if ln.startswith("req abc123")]
    assert len(req) == 1
    m = re.match(r"req abc123 slot=(\d+) prompt=300 cached=0 new=(\d+) finish=stop queue=\d+ms prefill=\d+ms \(\d+ tok/s\) decode=[\d.]+ tok/s$", req[0])
    assert m and int(m.group(2)) == r.emitted
    st = [ln for ln in logs if ln.startswith("stats:")]
    assert st and re.search(r"\d+ running, \d+ prefilling, \d+ waiting; [\d.]+ tok/s; \d+ done, \d+ failed; step [\d.]+ ms; prompt tokens from cache \d+%", st[0])


def test_event_loop_stays_responsive_while_the_engine_is_busy():
    """Engine calls run on the scheduler's thread: with every generate step taking 200 ms, /health and /tokenize still
    answer well within a step while a completion is being generated."""
    srv, sched, eng, pr = make_server("eight tk", step_seconds=0.2)

    async def fn(c):
        job = asyncio.ensure_future(c.post("/v1/chat/completions", json={"messages": MSG}))
        await asyncio.sleep(0.3)                       # the generation is under way
        worst = 0.0
        for _ in range(10):
            t0 = time.time()
            r = await c.get("/health")
            assert r.status == 200
            r = await c.post("/tokenize", json={"prompt": "hello there"})
            assert r.status == 200
            worst = max(worst, time.time() - t0)
            await asyncio.sleep(0.02)
        assert not job.done()                          # still generating: the probes ran alongside it
        out = await (await job).json()
        return worst, out
    worst, out = with_client(srv, fn)
    assert out["choices"][0]["finish_reason"] == "stop"
    assert worst < 0.1, f"a probe took {worst * 1e3:.0f} ms while the engine stepped"
    sched.shutdown()


def test_token_arrays_are_marshalled_once():
    """The prompt's int32 array is built on first use and reused by every later engine call on the same tokens."""
    from qwserve.engine import Tokens
    t = Tokens(range(50000))
    t0 = time.time()
    a = t.array()
    first = time.time() - t0
    t0 = time.time()
    for _ in range(100):
        assert t.array() is a
    again = (time.time() - t0) / 100
    assert again < first / 20 and a[49999] == 49999 and len(a) == 50000
    t.append(7)                                         # a changed list is marshalled again
    b = t.array()
    assert b is not a and len(b) == 50001 and b[50000] == 7


def test_cancelled_requests_leave_at_every_stage():
    """A request cancelled while it waits, while its prompt goes in (even when shorter prompts are ahead of it) or while it
    generates ends with "abort" and gives its slot back; the others are not disturbed."""
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    srv, sched, eng, pr = make_server("ok", slots=(8192, 8192), piece=256, start=False)
    eng.reply = lambda prompt: [66] * 50
    ends = {}

    def req(name, n, max_new=8):
        r = Request(tokens=Tokens([65] * n), max_new=max_new, sampling=Sampling(), stop_ids=[eng.eos], rid=name)
        r.on_done = lambda reason, name=name: ends.setdefault(name, reason)
        return r
    long_r, short_r, waiting_r = req("long", 4000), req("short", 600), req("waiting", 100)
    for r in (long_r, short_r, waiting_r):
        sched.submit(r)
    sched._drain_inbox()
    sched._admit()                                            # two slots: long and short are admitted, the third waits
    assert [r.rid for r in sched.prefilling] == ["long", "short"] and [r.rid for r in sched.waiting] == ["waiting"]
    sched._prefill()                                          # the shorter prompt goes first
    assert eng.prefill_order == [short_r.slot]
    sched.cancel(long_r)                                      # cancelled while a shorter prompt is still ahead of it
    sched.cancel(waiting_r)
    sched._prefill()
    assert ends["long"] == "abort" and not eng.busy[long_r.slot] and [r.rid for r in sched.prefilling] == ["short"]
    sched._admit()
    assert ends["waiting"] == "abort" and not sched.waiting
    while sched.prefilling:
        sched._prefill()
    assert [r.rid for r in sched.running] == ["short"]
    sched._step()
    sched.cancel(short_r)
    sched._step()
    assert ends["short"] == "abort" and not sched.running and eng.busy == [False, False]
    assert sched.stats["failed"] == 0


def test_a_client_that_goes_away_frees_its_slot():
    """A streaming client closes the connection mid-answer: the request is cancelled, its slot comes back, and the next
    request is served."""
    srv, sched, eng, pr = make_server("</think>" + "word " * 400, slots=(8192,), step_seconds=0.01)

    async def fn(c):
        r = await c.post("/v1/chat/completions", json={"messages": MSG, "stream": True, "max_tokens": 4000})
        got = 0
        async for line in r.content:
            if line.startswith(b"data: "):
                got += 1
            if got >= 5:
                break
        r.close()                                           # the client goes away in the middle of the answer
        t0 = time.time()
        while eng.busy[0] and time.time() - t0 < 5:
            await asyncio.sleep(0.05)
        freed = not eng.busy[0]
        nxt = await (await c.post("/v1/chat/completions", json={"messages": MSG, "max_tokens": 6})).json()
        return freed, nxt
    freed, nxt = with_client(srv, fn)
    assert freed and nxt["choices"][0]["finish_reason"] == "length" and nxt["usage"]["completion_tokens"] == 6
    assert sched.counts()["failed"] == 0
    sched.shutdown()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_scheduler_soak_with_injected_failures(seed):
    """Sixty requests of mixed sizes on three slots with failures injected at random: prompts the engine refuses, steps
    that raise for one slot, clients that cancel.  Every request ends exactly once, every slot comes back, the scheduler
    thread survives, and the requests nothing was done to end normally."""
    import random
    from qwserve.engine import Sampling, Tokens
    from qwserve.scheduler import Request
    rnd = random.Random(seed)
    srv, sched, eng, pr = make_server("ok", slots=(4096, 2048, 2048), piece=256, drafts=rnd.choice([0, 2]))
    eng.reply = lambda prompt: [66 + len(prompt) % 7] * 30
    eng.poison = 13
    ends, lock = {}, threading.Lock()
    reqs = []
    for i in range(60):
        n = rnd.choice([10, 100, 300, 900, 1800])
        toks = [65] * n
        fate = rnd.choices(["ok", "poison", "cancel", "step_error"], weights=[6, 1, 2, 1])[0]
        if fate == "poison":
            toks[rnd.randrange(n)] = 13
        r = Request(tokens=Tokens(toks), max_new=rnd.randrange(1, 25), sampling=Sampling(), stop_ids=[eng.eos], rid=f"r{i}")

        def done(reason, i=i):
            with lock:
                ends.setdefault(i, []).append(reason)
        r.on_done = done
        reqs.append((r, fate))
    for r, fate in reqs:
        sched.submit(r)
        if rnd.random() < 0.3:
            time.sleep(0.002)
    t0 = time.time()
    while len(ends) < len(reqs) and time.time() - t0 < 30:
        for r, fate in reqs:
            if fate == "cancel" and not r.cancelled and rnd.random() < 0.05:
                sched.cancel(r)
            if fate == "step_error" and r.slot >= 0 and r.prefill_done and not r.finish and not r.error and r.slot not in eng.generate_error:
                eng.generate_error[r.slot] = "injected failure"
        for s_ in list(eng.generate_error):                       # the failure is a one-off: clear it once its request has ended
            if not any(r.slot == s_ and not (r.finish or r.error) for r, _ in reqs):
                eng.generate_error.pop(s_, None)
        time.sleep(0.005)
    for r, fate in reqs:
        if fate == "cancel":
            sched.cancel(r)
    t0 = time.time()
    while len(ends) < len(reqs) and time.time() - t0 < 10:
        time.sleep(0.01)
    assert len(ends) == len(reqs) and all(len(v) == 1 for v in ends.values()), {k: v for k, v in ends.items() if len(v) != 1}
    assert sched.thread.is_alive() and sched.health() is None
    t0 = time.time()
    while any(eng.busy) and time.time() - t0 < 2:
        time.sleep(0.01)
    assert eng.busy == [False, False, False]
    for i, (r, fate) in enumerate(reqs):
        reason = ends[i][0]
        if fate == "ok":
            assert reason in ("stop", "length"), (i, reason)
        elif fate == "poison":
            assert reason.startswith("error: poisoned prompt")
        elif fate == "cancel":
            assert reason in ("abort", "stop", "length")          # it may have finished before the cancel arrived
    c = sched.counts()
    assert c["completed"] + c["failed"] >= 40 and c["running"] == 0 and c["waiting"] == 0 and c["prefilling"] == 0
    sched.shutdown()
