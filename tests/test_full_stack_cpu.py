"""The whole host stack on CPU: HTTP -> scheduler -> the server's ctypes binding -> libqw_engine.so -> CApi -> the real
Session (native planner, block store, chunker) -> a rule-based engine.  Speculative serving returns the text of plain
serving, a repeated prompt is served from the slot's snapshot, concurrent requests do not disturb one another."""
import asyncio

import pytest

from rule_engine import RuleEngine, make_session
from server_fixtures import make_prompter

aiohttp = pytest.importorskip("aiohttp")
from aiohttp.test_utils import TestClient, TestServer  # noqa: E402

MSG = [{"role": "user", "content": "tell me something"}]


def serve(monkeypatch, drafts, wrong=lambda pos: False, slots=3):
    from qwb200 import capi_impl
    from qwb200.native import build as nbuild
    from qwserve import engine as E
    from qwserve.api import Server
    from qwserve.scheduler import Scheduler
    nbuild.build()
    rule = RuleEngine(vocab=512, modulus=256, slots=slots, wrong=wrong)
    holder = {}

    def build_ops(o, rank, world, port):
        holder["ses"] = make_session(monkeypatch, rule, host_cache_bytes=8 << 20)
        return capi_impl.SessionOps(holder["ses"], None)
    monkeypatch.setattr(capi_impl, "build_ops", build_ops)
    eng = E.Engine({"synthetic": "tiny"}, nbuild.ENGINE_LIB)
    pr = make_prompter()
    sched = Scheduler(eng, drafts=drafts, prefill_piece=512, log=lambda *_: None)
    srv = Server(eng, pr, sched, "qw-rule")
    sched.start(watchdog=False)
    return srv, sched, eng, rule, holder


def with_client(srv, fn):
    from qwserve.api import make_app

    async def go():
        async with TestClient(TestServer(make_app(srv, dashboard=False))) as c:
            return await fn(c)
    return asyncio.run(go())


def chat(c, **kw):
    body = {"messages": MSG, "max_tokens": 40, "temperature": 0, "chat_template_kwargs": {"enable_thinking": False}}
    body.update(kw)
    return c.post("/v1/chat/completions", json=body)


def test_speculative_serving_equals_plain_serving(monkeypatch):
    texts = {}
    for drafts, wrong in ((0, lambda p: False), (3, lambda p: False), (3, lambda p: p % 4 == 0)):
        srv, sched, eng, rule, holder = serve(monkeypatch, drafts, wrong)

        async def fn(c):
            r = await chat(c)
            assert r.status == 200
            return await r.json()
        out = with_client(srv, fn)
        sched.shutdown()
        eng.close()
        ch = out["choices"][0]
        assert ch["finish_reason"] == "length" and out["usage"]["completion_tokens"] == 40
        texts[(drafts, wrong(4))] = ch["message"]["content"]
        if drafts:
            assert rule.draft_calls > 0 and max(max(r) for r in rule.verify_rows) > 1          # drafts really ran through the C ABI
    assert len(set(texts.values())) == 1 and len(next(iter(texts.values()))) > 0


def test_repeated_prompt_and_concurrent_requests(monkeypatch):
    srv, sched, eng, rule, holder = serve(monkeypatch, drafts=2)

    async def fn(c):
        a = await (await chat(c)).json()
        fed = rule.fed
        b = await (await chat(c)).json()                       # the same prompt again: nothing of it is fed a second time
        refed = rule.fed - fed - b["usage"]["completion_tokens"]
        rs = await asyncio.gather(*[chat(c, messages=[{"role": "user", "content": f"question number {i}"}], max_tokens=16 + i) for i in range(3)])
        many = [await r.json() for r in rs]
        solo = []
        for i in range(3):
            solo.append(await (await chat(c, messages=[{"role": "user", "content": f"question number {i}"}], max_tokens=16 + i)).json())
        await asyncio.sleep(1.3)                               # the scheduler refreshes the cache counters once a second
        health = await (await c.get("/health")).json()
        return a, b, refed, many, solo, health
    a, b, refed, many, solo, health = with_client(srv, fn)
    sched.shutdown()
    eng.close()
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] == b["usage"]["prompt_tokens"] and refed <= 0
    for m, s_, i in zip(many, solo, range(3)):
        assert m["choices"][0]["message"]["content"] == s_["choices"][0]["message"]["content"]      # batched with others == alone
        assert m["usage"]["completion_tokens"] == 16 + i
    assert health["status"] == "ok" and health["prefix_cache"]["prompt_tokens"] > 0 and health["prefix_cache"]["reused_tokens"] > 0
    assert health["decode"]["completed"] == 8 and health["decode"]["failed"] == 0


def test_stop_token_and_streaming_through_the_stack(monkeypatch):
    """The rule predicts the end-of-message token from the row of position 70 on: the answer stops there (drafts past it are dropped),
    and the streamed frames add up to the non-streamed answer."""
    import json
    srv, sched, eng, rule, holder = serve(monkeypatch, drafts=3)
    rule.stop_after, rule.stop_token = 70, make_prompter().token_id("<|im_end|>")

    async def fn(c):
        plain = await (await chat(c, max_tokens=200)).json()
        r = await chat(c, max_tokens=200, stream=True, messages=[{"role": "user", "content": "tell me something else"}])
        text, finish = "", None
        async for line in r.content:
            line = line.decode().strip()
            if line.startswith("data: ") and line != "data: [DONE]":
                f = json.loads(line[6:])
                if f.get("choices"):
                    text += f["choices"][0]["delta"].get("content") or ""
                    finish = f["choices"][0].get("finish_reason") or finish
        again = await (await chat(c, max_tokens=200, messages=[{"role": "user", "content": "tell me something else"}])).json()
        return plain, text, finish, again
    plain, text, finish, again = with_client(srv, fn)
    sched.shutdown()
    eng.close()
    ch = plain["choices"][0]
    assert ch["finish_reason"] == "stop" and 0 < plain["usage"]["completion_tokens"] < 60
    # the row of position 70 is the first that predicts the stop token, which then sits at position 71 and ends the answer
    assert plain["usage"]["prompt_tokens"] + plain["usage"]["completion_tokens"] == 72
    assert finish == "stop" and text == again["choices"][0]["message"]["content"]


def test_soak_many_requests_shared_prefixes_unreliable_drafts(monkeypatch):
    """Thirty requests at once on three slots: a long shared system prompt (restored from the block store into whichever
    slot comes free), prompts of several lengths, drafts that are wrong at pseudo-random positions, a few clients that
    go away.  Every answer equals the answer of the same request served alone without drafts, and every slot's state
    stays the state of the tokens it holds."""
    import random
    rnd = random.Random(11)
    system = "You are a careful assistant. " * 40                     # ~1,200 byte tokens: four full blocks and a bit
    reqs = []
    for i in range(30):
        msgs = ([{"role": "system", "content": system}] if i % 3 else []) + [{"role": "user", "content": f"request {i}: " + "x" * rnd.randrange(0, 300)}]
        reqs.append(dict(messages=msgs, max_tokens=rnd.randrange(4, 50)))

    def run(drafts, wrong, concurrent, drop=()):
        srv, sched, eng, rule, holder = serve(monkeypatch, drafts, wrong)

        async def one(c, i, r):
            if i in drop:                                          # a client that leaves after the first frames
                resp = await chat(c, stream=True, **r)
                n = 0
                async for line in resp.content:
                    n += line.startswith(b"data: ")
                    if n >= 2:
                        break
                resp.close()
                return None
            return (await (await chat(c, **r)).json())["choices"][0]["message"]["content"]

        async def fn(c):
            if concurrent:
                return await asyncio.gather(*[one(c, i, r) for i, r in enumerate(reqs)])
            return [await one(c, i, r) for i, r in enumerate(reqs)]
        out = with_client(srv, fn)
        import time
        t0 = time.time()
        while any(s_.busy for s_ in holder["ses"].slots) and time.time() - t0 < 5:
            time.sleep(0.05)
        stats = holder["ses"].cache_stats()
        ok = all(rule.consistent(s, rule.slot[s].tokens) for s in range(3))
        busy = [s_.busy for s_ in holder["ses"].slots]
        sched.shutdown()
        eng.close()
        return out, stats, ok, busy, rule
    want, _, ok0, _, _ = run(0, lambda p: False, concurrent=False)
    got, stats, ok1, busy, rule = run(4, lambda p: (p * 2654435761) % 7 < 2, concurrent=True, drop={5, 17})
    assert ok0 and ok1 and busy == [False, False, False]
    for i, (g, w) in enumerate(zip(got, want)):
        if i not in (5, 17):
            assert g == w, i
    assert stats["reused_tokens"] >= 1024 and stats["hits"] >= 1 and rule.draft_calls > 0


def test_a_step_that_fails_half_way_fails_its_batch_and_nothing_else(monkeypatch):
    """The engine raises in the middle of a step, after one request's rows were kept: the requests of that step end with
    an error (none is retried: its pending token may have been decoded already), their slots come back, and the same
    prompts served again afterwards give the answers of an undisturbed server."""
    srv, sched, eng, rule, holder = serve(monkeypatch, drafts=2)
    rule.fail_accept_at = 6
    prompts = [[{"role": "user", "content": f"case {i} " + "y" * (40 * i)}] for i in range(3)]

    async def fn(c):
        first = await asyncio.gather(*[chat(c, messages=m, max_tokens=30) for m in prompts])
        first = [(r.status, await r.json()) for r in first]
        again = [await (await chat(c, messages=m, max_tokens=30)).json() for m in prompts]
        health = await (await c.get("/health")).json()
        return first, again, health
    first, again, health = with_client(srv, fn)
    busy = [s_.busy for s_ in holder["ses"].slots]
    ok = all(rule.consistent(s, rule.slot[s].tokens) for s in range(3))
    sched.shutdown()
    eng.close()
    failed = [st for st, body in first if st != 200 or "error" in body]
    assert failed and all(st == 500 for st, _ in first if st != 200)
    assert "step failed after slot state changed" in json_of(first)
    assert busy == [False, False, False] and ok and health["status"] == "ok"
    # an undisturbed server gives the reference answers
    srv2, sched2, eng2, rule2, _ = serve(monkeypatch, drafts=0)

    async def fn2(c):
        return [await (await chat(c, messages=m, max_tokens=30)).json() for m in prompts]
    want = with_client(srv2, fn2)
    sched2.shutdown()
    eng2.close()
    assert [a["choices"][0]["message"]["content"] for a in again] == [w["choices"][0]["message"]["content"] for w in want]


def json_of(first):
    import json
    return json.dumps([b for _, b in first])


def test_logprobs_through_the_stack(monkeypatch):
    """``logprobs`` with ``top_logprobs``: every emitted token comes with its log-probability and the most likely tokens of
    its row - the row index the session reports for a speculative step must be the row the token was drawn from, so the
    first alternative is the token itself (the draw is greedy here) with the same log-probability."""
    srv, sched, eng, rule, holder = serve(monkeypatch, drafts=3, wrong=lambda p: p % 5 == 0)
    rule.spread = True

    async def fn(c):
        return await (await chat(c, max_tokens=24, logprobs=True, top_logprobs=3)).json()
    out = with_client(srv, fn)
    sched.shutdown()
    eng.close()
    entries = out["choices"][0]["logprobs"]["content"]
    assert len(entries) == 24
    for e in entries:
        top = e["top_logprobs"]
        assert len(top) == 3 and top[0]["token"] == e["token"] and abs(top[0]["logprob"] - e["logprob"]) < 1e-4
        assert top[0]["logprob"] >= top[1]["logprob"] >= top[2]["logprob"] and e["logprob"] < 0


def test_forced_end_of_reasoning_through_the_stack(monkeypatch):
    """A model that never stops reasoning, a budget of eight tokens: the closing tokens are fed as given (each by a plain
    one-token step whose own draw is dropped), the answer follows, and the slot holds exactly what was emitted."""
    srv, sched, eng, rule, holder = serve(monkeypatch, drafts=3)
    pr = make_prompter()

    async def fn(c):
        body = {"messages": MSG, "max_tokens": 40, "temperature": 0, "thinking_budget": 8}
        return await (await c.post("/v1/chat/completions", json=body)).json()
    out = with_client(srv, fn)
    held = [list(rule.slot[s].tokens) for s in range(3) if rule.slot[s].tokens]
    ok = all(rule.consistent(s, rule.slot[s].tokens) for s in range(3))
    sched.shutdown()
    eng.close()
    m = out["choices"][0]["message"]
    close = pr.encode("\n</think>\n\n")
    assert out["usage"]["completion_tokens"] == 40 and out["usage"]["completion_tokens_details"]["reasoning_tokens"] >= 8
    assert m["reasoning_content"] and m["content"] and ok and len(held) == 1
    toks = held[0]
    at = next(i for i in range(len(toks)) if toks[i:i + len(close)] == close)          # the forced tokens are in the slot, in order
    think_open = pr.token_id("<think>")
    opened = max(i for i, t in enumerate(toks[:at]) if t == think_open)
    assert 8 <= at - opened - 1 <= 8 + 3 + 1                                             # the budget, plus at most one speculative step's overshoot
