"""Continuous-batching scheduler: one thread that is the only caller of the engine's C API.

Each loop iteration admits waiting requests into free slots (arrival order, without head-of-line blocking: a
request that does not fit is skipped, and retried only after a release), advances prompts that are still
being prefilled by one piece each while giving decoding its share of the time, and runs one generation step
for up to ``max_step`` requests round-robin.  A request failing inside the engine fails alone; a failed
engine, a dead scheduler thread or an engine call that hangs make ``health()`` report unhealthy, and the
watchdog then exits the process so that a supervisor restarts it
(reference behaviour: server/qwserve/scheduler.py:54-580)."""
from __future__ import annotations

import collections
import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

from .engine import Sampling, Tokens

QW_STEP_LOGITS = 1


@dataclass
class Request:
    tokens: Tokens
    max_new: int
    sampling: Sampling
    stop_ids: List[int] = field(default_factory=list)
    logprobs: int = 0                    # top-k logprobs per token (0 = none)
    thinking_budget: int = 0             # tokens of reasoning before the closing tokens are forced (0 = unlimited)
    think_open: int = -1
    think_close_id: int = -1
    think_close: List[int] = field(default_factory=list)   # tokens fed when the budget is spent (e.g. "\n</think>\n\n")
    start_in_think: bool = False
    rid: str = "-"
    media: list = field(default_factory=list)
    on_token: Optional[Callable[[int, float, Optional[list]], None]] = None
    on_done: Optional[Callable[[str], None]] = None        # finish reason or error text
    # ---- filled by the scheduler
    slot: int = -1
    pending: int = -1
    emitted: int = 0
    reused: int = 0
    reasoning: int = 0
    in_think: bool = False
    cancelled: bool = False
    no_slot: bool = False
    t_submit: float = field(default_factory=time.time)
    load_deadline: float = 0.0          # until when the request waits for its stored prefix to be read from disk
    t_admit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    error: str = ""
    finish: str = ""
    prefill_done: bool = False

    def timings(self) -> dict:
        """llama.cpp-style timings object."""
        pre = max(1e-9, self.t_first - self.t_admit)
        gen = max(1e-9, self.t_done - self.t_first)
        n_prompt = len(self.tokens) - self.reused
        return {"cache_n": self.reused, "prompt_n": n_prompt, "prompt_ms": pre * 1e3, "prompt_per_second": n_prompt / pre,
                "predicted_n": self.emitted, "predicted_ms": gen * 1e3, "predicted_per_second": self.emitted / gen,
                "queue_ms": (self.t_admit - self.t_submit) * 1e3}


class Scheduler:
    def __init__(self, engine, drafts: int = 0, prefill_piece: int = 2048, decode_share: float = 0.25, max_step: int = 16,
                 stuck_seconds: float = 300.0, exit_grace: float = 30.0, log_interval: float = 30.0, log=print,
                 share_min: int = 1024, share_wait: float = 30.0, load_wait: float = 30.0):
        self.e, self.k = engine, drafts if getattr(engine, "has_mtp", False) else 0
        self.piece, self.decode_share, self.max_step = prefill_piece, decode_share, max_step
        self.max_batch_prefill = 8          # short prompts prefilled by one engine call
        self.stuck_seconds, self.exit_grace, self.log = stuck_seconds, exit_grace, log
        self.log_interval, self._logged_at, self._logged_tokens = log_interval, time.time(), 0
        # A request whose prompt shares at least `share_min` tokens with one that is being prefilled waits (at most `share_wait`
        # seconds) until that one is in, so that it restores the shared part from the prefix cache instead of computing it
        # a second time; blocks that are only on disk are read in the background for at most `load_wait` seconds before the
        # prompt begins (QW_SHARE_MIN / QW_SHARE_WAIT of the reference's scheduler, server/qwserve/scheduler.py:315-398).
        self.share_min, self.share_wait, self.load_wait = share_min, share_wait, load_wait
        self.loading: List[Request] = []
        self.inbox: "queue.Queue[Request]" = queue.Queue()
        self.waiting: Deque[Request] = collections.deque()
        self.prefilling: List[Request] = []
        self.running: List[Request] = []
        self.stop_flag = threading.Event()
        self.released = True
        self.call_started = 0.0           # start of the engine call in flight (0 = none)
        self.stats = collections.Counter()
        self.rr = 0
        self.thread = threading.Thread(target=self._loop, name="qw-scheduler", daemon=True)
        self.watchdog: Optional[threading.Thread] = None
        self.unhealthy_since = 0.0
        self._cache_stats: dict = {}
        self._stats_at = 0.0

    # ---- public
    def start(self, watchdog: bool = True):
        self.thread.start()
        if watchdog:
            self.watchdog = threading.Thread(target=self._watch, name="qw-watchdog", daemon=True)
            self.watchdog.start()

    def submit(self, r: Request):
        r.in_think = r.start_in_think
        self.inbox.put(r)

    def cancel(self, r: Request):
        """Called from any thread (client went away): the scheduler drops the request at its next look."""
        r.cancelled = True

    @property
    def cache_stats(self) -> dict:
        return self._cache_stats

    def counts(self) -> dict:
        return {"waiting": len(self.waiting) + self.inbox.qsize(), "prefilling": len(self.prefilling) + len(self.loading), "running": len(self.running),
                **{k: self.stats[k] for k in ("completed", "failed", "tokens", "steps")}, "step_ms": 1e3 * self.stats.get("step_s", 0.0)}

    def shutdown(self):
        self.stop_flag.set()
        self.thread.join(timeout=10)

    def health(self) -> Optional[str]:
        """None while healthy, else the reason."""
        f = self.e.failure()
        if f:
            return "engine failure: " + f
        if not self.thread.is_alive() and not self.stop_flag.is_set():
            return "scheduler thread died"
        t = self.call_started
        if t and time.time() - t > self.stuck_seconds:
            return f"engine call running for {time.time() - t:.0f} s"
        return None

    # ---- engine calls are bracketed so a hang is visible to health()
    def _call(self, fn, *a):
        self.call_started = time.time()
        try:
            return fn(*a)
        finally:
            self.call_started = 0.0

    def _watch(self):
        while not self.stop_flag.wait(1.0):
            reason = self.health()
            if reason is None:
                self.unhealthy_since = 0.0
                continue
            if not self.unhealthy_since:
                self.unhealthy_since = time.time()
                self.log(f"unhealthy: {reason}")
            elif time.time() - self.unhealthy_since > self.exit_grace:
                self.log(f"exiting after {self.exit_grace:.0f} s unhealthy: {reason}")
                os._exit(3)

    # ---- loop
    def _loop(self):
        while not self.stop_flag.is_set():
            if time.time() - self._stats_at > 1.0:
                self._stats_at = time.time()
                try:
                    self._cache_stats = self.e.cache_stats()
                except Exception:
                    pass
                self._stats_line()
            busy = self._drain_inbox()
            busy |= self._admit()
            busy |= self._poll_loads()
            t0 = time.time()
            busy |= self._prefill()
            spent = time.time() - t0
            if self.running:
                # decoding gets at least its share of the time a prefill piece took
                steps = max(1, int(spent * self.decode_share / max(1e-3, self.stats.get("step_s", 0.02)))) if spent else 1
                for _ in range(steps):
                    if not self.running:
                        break
                    self._step()
                busy = True
            if not busy:
                try:
                    self.waiting.append(self.inbox.get(timeout=0.05))
                except queue.Empty:
                    pass

    def _stats_line(self):
        """Every ``log_interval`` seconds while there is work: queue depth, throughput, prefix-cache reuse."""
        now = time.time()
        if self.log_interval <= 0 or now - self._logged_at < self.log_interval:
            return
        c = self.counts()
        tok = c["tokens"] + sum(r.emitted for r in self.running)
        if tok != self._logged_tokens or c["waiting"] or c["prefilling"] or c["running"]:
            cs = self._cache_stats or {}
            reuse = 100.0 * cs.get("reused_tokens", 0) / max(1, cs.get("prompt_tokens", 0))
            self.log(f"stats: {c['running']} running, {c['prefilling']} prefilling, {c['waiting']} waiting; "
                     f"{(tok - self._logged_tokens) / (now - self._logged_at):.1f} tok/s; {c['completed']} done, {c['failed']} failed; "
                     f"step {c['step_ms']:.1f} ms; prompt tokens from cache {reuse:.0f}%")
        self._logged_at, self._logged_tokens = now, tok

    def _drain_inbox(self) -> bool:
        got = False
        while True:
            try:
                self.waiting.append(self.inbox.get_nowait())
                got = True
            except queue.Empty:
                return got

    def _fail(self, r: Request, msg: str):
        r.error, r.t_done = msg, time.time()
        self.stats["failed"] += 1
        if r.slot >= 0:
            try:
                self.e.release(r.slot)
            except Exception:
                pass
            r.slot = -1
            self.released = True
        if r.on_done:
            r.on_done("error: " + msg)

    def _admit(self) -> bool:
        if not self.waiting:
            return False
        retry, self.released = self.released, False
        admitted = False
        keep: Deque[Request] = collections.deque()
        while self.waiting:
            r = self.waiting.popleft()
            if r.cancelled:
                r.finish = "abort"
                if r.on_done:
                    r.on_done("abort")
                continue
            if r.no_slot and not retry:                   # it found no slot before and none was released since
                keep.append(r)
                continue
            if self._shares_prefix_in_flight(r):
                keep.append(r)
                continue
            try:
                slot = self._call(self.e.acquire, r.tokens, r.max_new, r.media)
            except Exception as ex:                       # this request fails alone
                self._fail(r, str(ex))
                continue
            if slot < 0:
                r.no_slot = True
                keep.append(r)                            # no slot for it now: later arrivals may still fit
                continue
            r.slot, r.t_admit = slot, time.time()
            pending = False
            if hasattr(self.e, "prefetch"):
                try:
                    pending = bool(self._call(self.e.prefetch, slot, r.tokens, r.media))
                except Exception:
                    pending = False                       # a failed read-ahead only costs the time it would have saved
            if pending:
                r.load_deadline = time.time() + self.load_wait
                self.loading.append(r)
                admitted = True
                continue
            admitted = self._begin(r) or admitted
        self.waiting = keep
        return admitted

    def _begin(self, r: "Request") -> bool:
        try:
            r.reused = self._call(self.e.begin_prompt, r.slot, r.tokens, r.media)
            self._call(self.e.set_stop_tokens, r.slot, r.stop_ids)
        except Exception as ex:
            self._fail(r, str(ex))
            return False
        self.prefilling.append(r)
        return True

    def _poll_loads(self) -> bool:
        """Requests whose stored prefix is being read from disk begin once the reads are done (or took too long)."""
        if not self.loading:
            return False
        still, began = [], False
        for r in self.loading:
            if r.cancelled:
                self._call(self.e.release, r.slot)
                self.released = True
                r.finish = "abort"
                if r.on_done:
                    r.on_done("abort")
                continue
            try:
                pending = bool(self._call(self.e.prefetch, r.slot, r.tokens, r.media)) and time.time() < r.load_deadline
            except Exception:
                pending = False
            if pending:
                still.append(r)
            else:
                began = self._begin(r) or began
        self.loading = still
        return began

    def _shares_prefix_in_flight(self, r: "Request") -> bool:
        if self.share_min <= 0 or not self.prefilling or time.time() - r.t_submit > self.share_wait:
            return False
        n = len(r.tokens)
        if n < self.share_min:
            return False
        for p in self.prefilling:
            m = min(n, len(p.tokens))
            if m >= self.share_min and r.tokens[:self.share_min] == p.tokens[:self.share_min]:
                return True
        return False

    def _prefill(self) -> bool:
        if not self.prefilling:
            return False
        gone = [q for q in self.prefilling if q.cancelled]                 # wherever they stand in the order: their slots are needed
        for q in gone:
            self.prefilling.remove(q)
            q.finish = "abort"
            self._finish(q)
        if gone:
            return True
        self.prefilling.sort(key=lambda r: len(r.tokens) - r.reused)       # short prompts first
        r = self.prefilling[0]
        # several prompts whose uncached part fits one piece go in with one engine call (on several GPUs one round trip to
        # the worker ranks instead of one per prompt); reference: _batch, server/qwserve/scheduler.py:315-398
        short = [q for q in self.prefilling if not q.cancelled and len(q.tokens) - q.reused <= self.piece][:self.max_batch_prefill]
        if len(short) >= 2 and hasattr(self.e, "prefill_batch"):
            try:
                done = self._call(self.e.prefill_batch, [q.slot for q in short], [self.piece] * len(short))
            except Exception as ex:
                for q in short:                 # which slots advanced is unknown: none of these prompts is retried
                    self.prefilling.remove(q)
                    self._fail(q, str(ex))
                return True
            for q, d in zip(short, done):
                if d:
                    self._prompt_in(q)
            self.stats["batched_prefills"] += 1
            return True
        try:
            done = self._call(self.e.prefill_some, r.slot, self.piece)
            if done:
                self._prompt_in(r)
        except Exception as ex:
            if r in self.prefilling:
                self.prefilling.remove(r)
            self._fail(r, str(ex))
        return True

    def _prompt_in(self, r: "Request") -> None:
        """The prompt is in: sample its first token and move the request to the running set."""
        try:
            tok, lp = self._call(self.e.sample_prompt, r.slot, r.sampling)
            self.prefilling.remove(r)
            r.prefill_done, r.t_first = True, time.time()
            self._emit(r, [tok], [lp], -1, False)
            if not r.finish:
                self.running.append(r)
        except Exception as ex:
            if r in self.prefilling:
                self.prefilling.remove(r)
            self._fail(r, str(ex))

    def _emit(self, r: Request, toks, lps, first_row, stopped):
        for j, (t, lp) in enumerate(zip(toks, lps)):
            top = None
            if r.logprobs:
                try:
                    top = self.e.top_logprobs_prompt(r.slot, r.logprobs) if first_row < 0 else self.e.top_logprobs(first_row + j, r.logprobs)
                except Exception:
                    top = None
            r.emitted += 1
            r.pending = t
            if t == r.think_open:
                r.in_think = True
            elif t == r.think_close_id:
                r.in_think = False
            elif r.in_think:
                r.reasoning += 1
            if r.on_token:
                r.on_token(t, lp, top)
            if t in r.stop_ids:
                r.finish = "stop"
                break
            if r.emitted >= r.max_new:
                r.finish = "length"
                break
        if stopped and not r.finish:
            r.finish = "stop"
        if r.cancelled and not r.finish:
            r.finish = "abort"
        if r.finish:
            self._finish(r)
        elif r.in_think and r.thinking_budget and r.reasoning >= r.thinking_budget and r.think_close:
            self._close_thinking(r)

    def _close_thinking(self, r: Request):
        """The reasoning budget is spent: feed the closing tokens as given.  Each one costs a plain one-token
        step whose sampled token is dropped in favour of the forced one."""
        try:
            for f in r.think_close:
                self._call(self.e.generate, [(r.slot, r.pending, 1, 0, r.sampling)], 0)
                r.pending = f
                r.emitted += 1
                if r.on_token:
                    r.on_token(f, 0.0, None)
            r.in_think = False
            self.stats["forced_think_close"] += 1
            if r.emitted >= r.max_new:
                r.finish = "length"
                self._finish(r)
        except Exception as ex:
            if r in self.running:
                self.running.remove(r)
            self._fail(r, str(ex))

    def _finish(self, r: Request):
        r.t_done = time.time()
        if r in self.running:
            self.running.remove(r)
        try:
            self.e.release(r.slot)
        except Exception:
            pass
        self.released = True
        self.stats["completed"] += 1
        self.stats["tokens"] += r.emitted
        tm = r.timings()
        self.log(f"req {r.rid} slot={r.slot} prompt={len(r.tokens)} cached={r.reused} new={r.emitted} finish={r.finish} "
                 f"queue={tm['queue_ms']:.0f}ms prefill={tm['prompt_ms']:.0f}ms ({tm['prompt_per_second']:.0f} tok/s) "
                 f"decode={tm['predicted_per_second']:.1f} tok/s")
        if r.on_done:
            r.on_done(r.finish)

    def _step(self):
        n = min(self.max_step, len(self.running))
        batch = [self.running[(self.rr + i) % len(self.running)] for i in range(n)]
        self.rr = (self.rr + n) % max(1, len(self.running))
        reqs = []
        for r in [r for r in batch if r.cancelled]:
            batch.remove(r)
            r.finish = "abort"
            self._finish(r)
        if not batch:
            return
        for r in batch:
            reqs.append((r.slot, r.pending, max(1, r.max_new - r.emitted), QW_STEP_LOGITS if r.logprobs else 0, r.sampling))
        t0 = time.time()
        try:
            outs = self._call(self.e.generate, reqs, self.k)
        except Exception as ex:
            if len(batch) == 1 or "step failed after slot state changed" in str(ex):
                # a refusal of a single request, or a failure after the engine had already advanced some of the slots: repeating
                # the step for the others would decode their pending token twice, so the whole batch fails
                for r in batch:
                    self.running.remove(r)
                    self._fail(r, str(ex))
            else:                                          # the step was refused before anything ran: find the culprit one by one
                for r in batch:
                    try:
                        o = self._call(self.e.generate, [(r.slot, r.pending, max(1, r.max_new - r.emitted), 0, r.sampling)], self.k)
                        self._emit(r, *o[0])
                    except Exception as ex1:
                        self.running.remove(r)
                        self._fail(r, str(ex1))
            return
        dt = time.time() - t0
        self.stats["step_s"] = 0.9 * self.stats.get("step_s", dt) + 0.1 * dt
        self.stats["steps"] += 1
        for r, (toks, lps, row, stopped) in zip(batch, outs):
            self._emit(r, toks, lps, row, stopped)
