"""Smoke test of a running server, for deployments: health, model list, tokenizer round trip, one short chat completion
(streamed and not), and - with ``--follow-up`` - a second turn whose time to first token shows the prefix cache at work.

    python -m qwserve.smoke [--url http://127.0.0.1:8000] [--max-tokens 16] [--follow-up] [--timeout 120]

Exit code 0 when every check passed; the report (one JSON line) names the first check that did not.
(Role of the reference's scripts/prod-smoke.sh.)"""
import argparse
import asyncio
import json
import sys
import time


async def run_checks(session, base: str, max_tokens: int = 16, follow_up: bool = False) -> dict:
    rep = {"ok": False, "checks": []}

    def note(name, ok, **kw):
        rep["checks"].append({"name": name, "ok": bool(ok), **kw})
        return ok

    async with session.get(base + "/health") as r:
        body = await r.json()
        if not note("health", r.status == 200 and body.get("status") in ("ok", "healthy", "ready"), status=r.status, body=body):
            return rep
    async with session.get(base + "/v1/models") as r:
        body = await r.json()
        models = [m.get("id") for m in body.get("data", [])]
        if not note("models", r.status == 200 and len(models) >= 1, models=models):
            return rep
    model = models[0]
    async with session.post(base + "/tokenize", json={"model": model, "prompt": "hello world"}) as r:
        body = await r.json()
        if not note("tokenize", r.status == 200 and len(body.get("tokens", [])) >= 1, count=len(body.get("tokens", []))):
            return rep
    msgs = [{"role": "user", "content": "Say hello in one short sentence."}]
    t0 = time.time()
    async with session.post(base + "/v1/chat/completions", json={"model": model, "messages": msgs, "max_tokens": max_tokens}) as r:
        body = await r.json()
        ch = (body.get("choices") or [{}])[0]
        text = (ch.get("message") or {}).get("content")
        usage = body.get("usage") or {}
        if not note("chat", r.status == 200 and text is not None and usage.get("completion_tokens", 0) >= 1, seconds=round(time.time() - t0, 3),
                    finish=ch.get("finish_reason"), completion_tokens=usage.get("completion_tokens")):
            return rep
    t0, first, pieces = time.time(), None, 0
    async with session.post(base + "/v1/chat/completions", json={"model": model, "messages": msgs, "max_tokens": max_tokens, "stream": True}) as r:
        done = False
        async for line in r.content:
            line = line.decode().strip()
            if line == "data: [DONE]":
                done = True
            elif line.startswith("data: "):
                if first is None:
                    first = time.time() - t0
                pieces += 1
        if not note("chat_stream", r.status == 200 and done and pieces >= 1, ttft_s=round(first or -1, 3), frames=pieces):
            return rep
    if follow_up:
        msgs2 = msgs + [{"role": "assistant", "content": text or "Hello."}, {"role": "user", "content": "And again, shorter."}]
        t0, first = time.time(), None
        async with session.post(base + "/v1/chat/completions", json={"model": model, "messages": msgs2, "max_tokens": max_tokens, "stream": True}) as r:
            async for line in r.content:
                if first is None and line.decode().startswith("data: "):
                    first = time.time() - t0
            if not note("follow_up", r.status == 200 and first is not None, ttft_s=round(first or -1, 3)):
                return rep
    rep["ok"] = True
    return rep


async def amain(a) -> int:
    import aiohttp
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=a.timeout)) as s:
        try:
            rep = await run_checks(s, a.url.rstrip("/"), a.max_tokens, a.follow_up)
        except Exception as ex:          # noqa: BLE001 - a refused connection or a non-JSON answer is a failed smoke test
            rep = {"ok": False, "error": f"{type(ex).__name__}: {ex}"}
    print(json.dumps(rep), flush=True)
    return 0 if rep.get("ok") else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--follow-up", action="store_true")
    ap.add_argument("--timeout", type=float, default=120.0)
    sys.exit(asyncio.run(amain(ap.parse_args())))


if __name__ == "__main__":
    main()
