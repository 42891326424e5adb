"""OpenAI-compatible HTTP front end (aiohttp): chat completions (streaming and not, with reasoning / tool-call
routing, logprobs, usage and llama.cpp-style timings), text completions, models, tokenize and health
(reference behaviour: server/qwserve/api.py:25-352, server/qwserve/__main__.py:58-63).

All tokenising and template work runs in a small thread pool so that the event loop only moves bytes; the
scheduler thread hands tokens back through ``loop.call_soon_threadsafe`` into one asyncio queue per request."""
from __future__ import annotations

import asyncio
import concurrent.futures
import json
import time
import uuid
from typing import Any, Dict, List, Optional

from aiohttp import web

from .detok import IncrementalDetok
from .engine import Sampling, Tokens
from .output_parser import OutputParser, TagIds
from .prompt import Prompter, resolve_thinking
from .scheduler import Request, Scheduler
from .tool_calls import parse_tool_call


def _err(msg: str, status: int = 400, kind: str = "invalid_request_error"):
    return web.json_response({"error": {"message": msg, "type": kind}}, status=status)


# Sampling defaults of the model card, by mode; a request's own fields override them one by one.
DEFAULTS_THINKING = dict(temperature=1.0, top_p=0.95, top_k=20, min_p=0.0, presence_penalty=1.5)
DEFAULTS_PLAIN = dict(temperature=0.7, top_p=0.8, top_k=20, min_p=0.0, presence_penalty=1.5)


SAMPLING_FIELDS = ("temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty")


def model_sampling_defaults(model_dir: Optional[str]) -> Dict[str, float]:
    """The numeric sampling fields of the checkpoint's ``generation_config.json`` (none when the file is missing or
    unreadable).  They stand between the built-in defaults and a request's own fields, as vLLM does it
    (the reference: server/qwserve/scheduler.py:42-51)."""
    import os
    if not model_dir:
        return {}
    try:
        with open(os.path.join(model_dir, "generation_config.json")) as f:
            cfg = json.load(f)
    except (OSError, ValueError):
        return {}
    if not isinstance(cfg, dict):
        return {}
    return {k: cfg[k] for k in SAMPLING_FIELDS if isinstance(cfg.get(k), (int, float)) and not isinstance(cfg[k], bool)}


def sampling_of(body: Dict[str, Any], thinking: bool, model_defaults: Optional[Dict[str, float]] = None) -> Sampling:
    d = dict(DEFAULTS_THINKING if thinking else DEFAULTS_PLAIN)
    d.update(model_defaults or {})
    for k in SAMPLING_FIELDS:
        if body.get(k) is not None:
            d[k] = body[k]
    seed = body.get("seed")
    return Sampling(temperature=float(d["temperature"]), top_p=float(d["top_p"]), top_k=int(d["top_k"]), min_p=float(d["min_p"]),
                    presence_penalty=float(d.get("presence_penalty", 0.0)), frequency_penalty=float(d.get("frequency_penalty", 0.0)),
                    repetition_penalty=float(d.get("repetition_penalty", 1.0)),
                    seed=int(seed) if seed is not None else uuid.uuid4().int & 0x7FFFFFFFFFFFFFFF)


class Server:
    def __init__(self, engine, prompter: Prompter, sched: Scheduler, model_name: str, preprocessor=None,
                 default_effort: Optional[str] = None, default_budget: int = 0, max_new_default: int = 32768,
                 sampling_defaults: Optional[Dict[str, float]] = None):
        self.engine, self.prompter, self.sched, self.model_name = engine, prompter, sched, model_name
        self.sampling_defaults = dict(sampling_defaults or {})
        self.pre = preprocessor
        self.default_effort, self.default_budget, self.max_new_default = default_effort, default_budget, max_new_default
        self.pool = concurrent.futures.ThreadPoolExecutor(max_workers=4, thread_name_prefix="qw-prep")
        tid = prompter.token_id
        self.tags = TagIds(tid("<think>"), tid("</think>"), tid("<tool_call>"), tid("</tool_call>"))
        self.eos = [t for t in (tid("<|im_end|>"), tid("<|endoftext|>")) if t is not None]
        self.close_tokens = prompter.encode("\n</think>\n\n") if self.tags.think_close is not None else []
        self.started = time.time()

    # ---- helpers
    async def offload(self, fn, *a):
        return await asyncio.get_running_loop().run_in_executor(self.pool, fn, *a)

    @property
    def max_len(self) -> int:
        return int(max(self.engine.slot_capacity(s) for s in range(self.engine.num_slots())))

    def _prepare_chat(self, body):
        """Runs in the pool: render, tokenise, fetch + preprocess media, expand placeholders."""
        enabled, effort, budget = resolve_thinking(body, self.default_effort, self.default_budget)
        kw = dict(body.get("chat_template_kwargs") or {})
        kw.pop("enable_thinking", None)
        if effort:
            kw.setdefault("reasoning_effort", effort)
        text = self.prompter.render(body["messages"], tools=body.get("tools"), enable_thinking=enabled, **kw)
        ids = self.prompter.encode(text)
        media = []
        if self.pre is not None:
            from .vision import expand_placeholders, media_of_part
            for m in body["messages"]:
                if isinstance(m.get("content"), list):
                    for part in m["content"]:
                        item = media_of_part(self.pre, part)
                        if item is not None:
                            media.append(item)
            if media:
                if not getattr(self.engine, "has_vision", False):
                    raise ValueError("this model was loaded without a vision tower")
                ids = expand_placeholders(ids, media, self.prompter.tok)
        starts_thinking = enabled and text.rstrip().endswith("<think>")
        return ids, media, enabled, budget, starts_thinking

    def _stop_strings(self, body) -> List[str]:
        s = body.get("stop")
        if not s:
            return []
        return [s] if isinstance(s, str) else [x for x in s if isinstance(x, str) and x]

    def _make_request(self, ids, body, media, budget, starts_thinking, q, loop, rid) -> Request:
        n_new = body.get("max_completion_tokens") or body.get("max_tokens") or self.max_new_default
        n_new = max(1, min(int(n_new), self.max_len - len(ids)))
        thinking = starts_thinking

        def on_token(tok, lp, top):
            loop.call_soon_threadsafe(q.put_nowait, ("tok", (tok, lp, top)))

        def on_done(reason):
            loop.call_soon_threadsafe(q.put_nowait, ("end", reason))
        lp_k = 0
        if body.get("logprobs"):
            lp_k = max(1, min(20, int(body.get("top_logprobs") or 1))) if not isinstance(body["logprobs"], bool) or body.get("top_logprobs") else 1
        return Request(tokens=Tokens(ids), max_new=n_new, sampling=sampling_of(body, thinking, self.sampling_defaults), stop_ids=list(self.eos),
                       logprobs=lp_k, thinking_budget=budget, think_open=self.tags.think_open if self.tags.think_open is not None else -1,
                       think_close_id=self.tags.think_close if self.tags.think_close is not None else -1,
                       think_close=list(self.close_tokens), start_in_think=starts_thinking,
                       media=self._engine_media(media), on_token=on_token, on_done=on_done, rid=rid)

    def _engine_media(self, media):
        if not media:
            return []
        from .engine import Media
        import ctypes as C
        import numpy as np
        out = []
        for m in media:
            starts = np.asarray([s for s, _ in m.spans], np.int64)
            em = Media(hash=int.from_bytes(m.key, "little"), video=int(m.kind == "video"), t=m.grid[0], h=m.grid[1], w=m.grid[2],
                       patches=m.patches.ctypes.data_as(C.c_void_p), starts=starts.ctypes.data_as(C.c_void_p))
            em._keep = (m.patches, starts)           # the arrays must outlive the request
            out.append(em)
        return out

    # ---- routes
    async def health(self, _):
        reason = self.sched.health()
        body = {"status": "ok" if reason is None else "unhealthy", "decode": self.sched.counts(), "prefix_cache": self.sched.cache_stats,
                "uptime_s": time.time() - self.started}
        if reason:
            body["reason"] = reason
        return web.json_response(body, status=200 if reason is None else 503)

    async def models(self, _):
        return web.json_response({"object": "list", "data": [{"id": self.model_name, "object": "model", "created": int(self.started),
                                                              "owned_by": "qw", "max_model_len": self.max_len}]})

    async def tokenize(self, request):
        try:
            body = await request.json()
        except Exception:
            return _err("body is not JSON")

        def work():
            if "messages" in body:
                return self._prepare_chat(body)[0]
            p = body.get("prompt", "")
            return list(p) if isinstance(p, list) else self.prompter.encode(p)
        try:
            ids = await self.offload(work)
        except Exception as ex:
            return _err(str(ex))
        return web.json_response({"count": len(ids), "max_model_len": self.max_len, "tokens": ids})

    def _lp_entry(self, tok, lp, top):
        s = self.prompter.decode([tok])
        e = {"token": s, "logprob": lp, "bytes": list(s.encode())}
        e["top_logprobs"] = [{"token": self.prompter.decode([i]), "logprob": l, "bytes": list(self.prompter.decode([i]).encode())}
                             for i, l in (top or [])]
        return e

    async def chat(self, request):
        try:
            body = await request.json()
        except Exception:
            return _err("body is not JSON")
        if not isinstance(body.get("messages"), list) or not body["messages"]:
            return _err("messages must be a non-empty list")
        if int(body.get("n") or 1) != 1:
            return _err("n > 1 is not supported")
        try:
            ids, media, enabled, budget, starts_thinking = await self.offload(self._prepare_chat, body)
        except Exception as ex:
            return _err(str(ex))
        if len(ids) >= self.max_len:
            return _err(f"prompt of {len(ids)} tokens exceeds the context of {self.max_len}")
        rid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        loop, q = asyncio.get_running_loop(), asyncio.Queue()
        req = self._make_request(ids, body, media, budget, starts_thinking, q, loop, rid)
        stream = bool(body.get("stream"))
        want_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        stops = self._stop_strings(body)
        parser = OutputParser(self.tags, start_in_think=starts_thinking)
        detok = {ch: IncrementalDetok(self.prompter.decode) for ch in ("reasoning", "content")}
        text = {"reasoning": "", "content": ""}
        tool_calls: List[dict] = []
        logprobs: List[dict] = []
        finish, n_out = None, 0

        def frame(delta, fin=None, lp=None):
            return {"id": rid, "object": "chat.completion.chunk", "created": created, "model": self.model_name,
                    "choices": [{"index": 0, "delta": delta, "logprobs": lp, "finish_reason": fin}]}

        resp = None
        if stream:
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
            await resp.prepare(request)
            await resp.write(b"data: " + json.dumps(frame({"role": "assistant", "content": ""})).encode() + b"\n\n")
        self.sched.submit(req)
        sent_content = 0          # characters of content already streamed (stop strings hold some back)
        hold = max((len(s) for s in stops), default=0)
        try:
            while True:
                kind, payload = await q.get()
                if kind == "end":
                    finish = finish or payload
                    break
                if finish is not None:          # a stop string ended the text: drop what was still in flight
                    continue
                tok, lp, top = payload
                n_out += 1
                if tok in self.eos:
                    continue
                routed = parser.push(tok)
                # a tool call is complete when its closing tag arrives
                if tok == self.tags.tool_close and parser.tool_tokens:
                    call = parse_tool_call(self.prompter.decode(parser.tool_tokens[-1]), body.get("tools"))
                    if call is not None:
                        call["index"] = len(tool_calls)
                        tool_calls.append(call)
                        if stream:
                            await resp.write(b"data: " + json.dumps(frame({"tool_calls": [call]})).encode() + b"\n\n")
                if routed is None or routed.channel == "tool":
                    continue
                ch = routed.channel
                piece = detok[ch].push(tok)
                text[ch] += piece
                entry = self._lp_entry(tok, lp, top) if req.logprobs else None
                if entry:
                    logprobs.append(entry)
                cut = -1
                if ch == "content" and stops:
                    hits = [text["content"].find(s, max(0, sent_content - hold)) for s in stops]
                    hits = [h for h in hits if h >= 0]
                    if hits:
                        cut = min(hits)
                        text["content"] = text["content"][:cut]
                        finish = "stop"
                if stream:
                    if ch == "reasoning":
                        if piece:
                            await resp.write(b"data: " + json.dumps(frame({"reasoning_content": piece, "reasoning": piece})).encode() + b"\n\n")
                    else:
                        upto = len(text["content"]) if cut >= 0 else max(sent_content, len(text["content"]) - hold)
                        if upto > sent_content or entry:
                            d = {"content": text["content"][sent_content:upto]}
                            sent_content = max(sent_content, upto)
                            await resp.write(b"data: " + json.dumps(frame(d, lp={"content": [entry]} if entry else None)).encode() + b"\n\n")
                if cut >= 0:
                    self.sched.cancel(req)
        except (asyncio.CancelledError, ConnectionResetError):
            self.sched.cancel(req)
            raise
        if isinstance(finish, str) and finish.startswith("error:"):
            if stream:
                await resp.write(b"data: " + json.dumps({"error": {"message": finish[7:], "type": "server_error"}}).encode() + b"\n\n")
                await resp.write(b"data: [DONE]\n\n")
                return resp
            return _err(finish[7:], 500, "server_error")
        for ch in ("reasoning", "content"):
            text[ch] += detok[ch].flush()
        if finish == "abort":
            finish = "stop"
        if tool_calls and finish == "stop":
            finish = "tool_calls"
        usage = {"prompt_tokens": len(ids), "completion_tokens": n_out, "total_tokens": len(ids) + n_out,
                 "prompt_tokens_details": {"cached_tokens": int(req.reused)},
                 "completion_tokens_details": {"reasoning_tokens": parser.reasoning_tokens}}
        timings = req.timings() if req.t_first else None
        if stream:
            if sent_content < len(text["content"]):
                await resp.write(b"data: " + json.dumps(frame({"content": text["content"][sent_content:]})).encode() + b"\n\n")
            last = frame({}, fin=finish)
            if timings:
                last["timings"] = timings
            await resp.write(b"data: " + json.dumps(last).encode() + b"\n\n")
            if want_usage:
                await resp.write(b"data: " + json.dumps({"id": rid, "object": "chat.completion.chunk", "created": created,
                                                         "model": self.model_name, "choices": [], "usage": usage}).encode() + b"\n\n")
            await resp.write(b"data: [DONE]\n\n")
            await resp.write_eof()
            return resp
        for c in tool_calls:
            c.pop("index", None)
        msg = {"role": "assistant", "content": text["content"] if (text["content"] or not tool_calls) else None,
               "reasoning_content": text["reasoning"] or None, "reasoning": text["reasoning"] or None}
        if tool_calls:
            msg["tool_calls"] = tool_calls
        out = {"id": rid, "object": "chat.completion", "created": created, "model": self.model_name,
               "choices": [{"index": 0, "message": msg, "logprobs": {"content": logprobs} if req.logprobs else None, "finish_reason": finish}],
               "usage": usage}
        if timings:
            out["timings"] = timings
        return web.json_response(out)

    async def completions(self, request):
        try:
            body = await request.json()
        except Exception:
            return _err("body is not JSON")
        prompt = body.get("prompt", "")
        if isinstance(prompt, str):
            ids = await self.offload(self.prompter.encode, prompt)
        elif isinstance(prompt, list) and all(isinstance(t, int) for t in prompt):
            ids = list(prompt)
        else:
            return _err("prompt must be a string or a token list")
        if not ids:
            return _err("prompt is empty")
        if len(ids) >= self.max_len:
            return _err(f"prompt of {len(ids)} tokens exceeds the context of {self.max_len}")
        rid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        loop, q = asyncio.get_running_loop(), asyncio.Queue()
        req = self._make_request(ids, body, [], 0, False, q, loop, rid)
        stream = bool(body.get("stream"))
        stops = self._stop_strings(body)
        detok = IncrementalDetok(self.prompter.decode)
        text, sent, n_out, finish = "", 0, 0, None
        hold = max((len(s) for s in stops), default=0)

        def frame(t, fin=None, **extra):
            return {"id": rid, "object": "text_completion", "created": created, "model": self.model_name,
                    "choices": [{"index": 0, "text": t, "finish_reason": fin}], **extra}
        resp = None
        if stream:
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
            await resp.prepare(request)
        self.sched.submit(req)
        try:
            while True:
                kind, payload = await q.get()
                if kind == "end":
                    finish = finish or payload
                    break
                if finish is not None:
                    continue
                tok = payload[0]
                n_out += 1
                if tok in self.eos:
                    continue
                text += detok.push(tok)
                cut = -1
                hits = [h for h in (text.find(s, max(0, sent - hold)) for s in stops) if h >= 0]
                if hits:
                    cut = min(hits)
                    text, finish = text[:cut], "stop"
                    self.sched.cancel(req)
                upto = len(text) if cut >= 0 else max(sent, len(text) - hold)
                if stream and upto > sent:
                    await resp.write(b"data: " + json.dumps(frame(text[sent:upto])).encode() + b"\n\n")
                sent = max(sent, upto)
        except (asyncio.CancelledError, ConnectionResetError):
            self.sched.cancel(req)
            raise
        if isinstance(finish, str) and finish.startswith("error:"):
            if stream:
                await resp.write(b"data: " + json.dumps({"error": {"message": finish[7:]}}).encode() + b"\n\ndata: [DONE]\n\n")
                return resp
            return _err(finish[7:], 500, "server_error")
        text += detok.flush()
        finish = "stop" if finish == "abort" else finish
        usage = {"prompt_tokens": len(ids), "completion_tokens": n_out, "total_tokens": len(ids) + n_out,
                 "prompt_tokens_details": {"cached_tokens": int(req.reused)}}
        extra = {"usage": usage}
        if req.t_first:
            extra["timings"] = req.timings()
        if stream:
            await resp.write(b"data: " + json.dumps(frame(text[sent:], fin=finish, **extra)).encode() + b"\n\ndata: [DONE]\n\n")
            await resp.write_eof()
            return resp
        return web.json_response(frame(text, fin=finish, **extra))

    async def on_shutdown(self, _app):
        """Stop the scheduler, then write the prefix cache's RAM blocks to the disk tier."""
        self.sched.shutdown()
        try:
            await self.offload(self.engine.persist)
        except Exception:
            pass


def make_app(server: Server, dashboard: bool = True) -> web.Application:
    app = web.Application(client_max_size=256 << 20)
    app.router.add_get("/health", server.health)
    app.router.add_get("/v1/models", server.models)
    app.router.add_post("/tokenize", server.tokenize)
    app.router.add_post("/v1/chat/completions", server.chat)
    app.router.add_post("/v1/completions", server.completions)
    app.on_shutdown.append(server.on_shutdown)
    if dashboard:
        from .dashboard import attach
        attach(app, server)
    return app
