"""Stand-ins for the server tests: a byte-level tokenizer with the model's special tokens, a chat template, and a
fake engine with the Python interface of ``qwserve.engine.Engine`` whose failures can be injected from the
test (the scheduler and HTTP layers are tested without a GPU)."""
import os
import sys
import threading
import time

SERVER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "v620-inference-engine_b200", "server")
if SERVER not in sys.path:
    sys.path.insert(0, SERVER)

SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
            "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"]

TEMPLATE = (
    "{% if tools %}<|im_start|>system\n# Tools\n{% for t in tools %}{{ t | tojson }}\n{% endfor %}<|im_end|>\n{% endif %}"
    "{% for m in messages %}<|im_start|>{{ m.role }}\n"
    "{% if m.content is string %}{{ m.content }}{% else %}{% for p in m.content %}"
    "{% if p.type == 'text' %}{{ p.text }}{% elif 'image' in p.type %}<|vision_start|><|image_pad|><|vision_end|>{% endif %}"
    "{% endfor %}{% endif %}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% if enable_thinking %}<think>\n{% else %}<think>\n\n</think>\n\n{% endif %}{% endif %}")


def make_tokenizer():
    from tokenizers import AddedToken, Tokenizer, decoders, models, pre_tokenizers
    alphabet = sorted(pre_tokenizers.ByteLevel.alphabet())
    tok = Tokenizer(models.BPE(vocab={c: i for i, c in enumerate(alphabet)}, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens([AddedToken(s, special=True) for s in SPECIALS])
    return tok


def make_prompter():
    from qwserve.prompt import Prompter
    return Prompter(tokenizer=make_tokenizer(), template=TEMPLATE)


class FakeEngine:
    """Replies with ``reply(prompt_ids) -> list of token ids`` (then the stop token), one token per generate
    step, or ``1 + k`` when drafts are on.  Injectable: ``poison`` (a token id whose presence makes acquire
    raise), ``generate_error`` (slot -> message), ``generate_block`` (an Event the next generate waits on),
    ``failed_with`` (what failure() returns)."""
    has_mtp = False
    has_vision = False

    def __init__(self, reply, slots=(4096, 1024, 1024), eos=2, step_seconds=0.0):
        self.reply, self.caps, self.eos, self.step_seconds = reply, list(slots), eos, step_seconds
        self.busy = [False] * len(slots)
        self.script = {}
        self.pos = {}
        self.prompt_left = {}
        self.poison = None
        self.generate_error = {}
        self.generate_block = None
        self.failed_with = ""
        self.calls = []
        self.owner = None
        self.lock = threading.Lock()
        self.persisted = 0
        self.prefill_order = []

    def _enter(self, name):
        # the C API allows one caller: every call must come from the same thread
        me = threading.get_ident()
        if self.owner is None:
            self.owner = me
        assert self.owner == me, f"{name} called from a second thread"
        self.calls.append(name)

    def failure(self):
        return self.failed_with

    def num_slots(self):
        return len(self.caps)

    def slot_capacity(self, s):
        return self.caps[s]

    def cache_stats(self):
        return {"hits": 0, "reused_tokens": 0, "ram_bytes": 0, "disk_bytes": 0}

    def persist(self):
        self.persisted += 1

    def set_boundary_token(self, t):
        pass

    def acquire(self, tokens, max_new, media=()):
        self._enter("acquire")
        if self.poison is not None and self.poison in tokens:
            raise RuntimeError("poisoned prompt")
        need = len(tokens) + max_new
        best = -1
        for s, cap in enumerate(self.caps):            # the smallest free slot that holds the request
            if not self.busy[s] and cap >= need and (best < 0 or cap < self.caps[best]):
                best = s
        if best >= 0:
            self.busy[best] = True
        return best

    def release(self, s):
        self.busy[s] = False

    def begin_prompt(self, s, tokens, media=()):
        self._enter("begin_prompt")
        self.script[s] = list(self.reply(list(tokens))) + [self.eos]
        self.pos[s] = 0
        self.prompt_left[s] = len(tokens)
        return 0

    def prefill_some(self, s, n):
        self._enter("prefill_some")
        self.prefill_order.append(s)
        self.prompt_left[s] -= min(n, self.prompt_left[s])
        return self.prompt_left[s] == 0

    def prefill_batch(self, slots, max_tokens):
        self._enter("prefill_batch")
        out = []
        for s, n in zip(slots, max_tokens):
            self.prefill_order.append(s)
            self.prompt_left[s] -= min(n, self.prompt_left[s])
            out.append(self.prompt_left[s] == 0)
        return out

    def set_stop_tokens(self, s, ids):
        pass

    def _next(self, s):
        t = self.script[s][min(self.pos[s], len(self.script[s]) - 1)]
        self.pos[s] += 1
        return t

    def sample_prompt(self, s, sp):
        self._enter("sample_prompt")
        return self._next(s), -0.5

    def generate(self, reqs, k):
        self._enter("generate")
        if self.generate_block is not None:
            self.generate_block.wait()
        if self.step_seconds:
            time.sleep(self.step_seconds)
        for slot, *_ in reqs:
            if slot in self.generate_error:
                raise RuntimeError(self.generate_error[slot])
        out, row = [], 0
        for slot, pending, budget, flags, sp in reqs:
            toks = []
            for _ in range(min(budget, 1 + k)):
                t = self._next(slot)
                toks.append(t)
                if t == self.eos:
                    break
            out.append((toks, [-0.25] * len(toks), row, toks[-1] == self.eos))
            row += len(toks)
        return out

    def top_logprobs(self, row, k):
        return [(65 + i, -1.0 - i) for i in range(k)]

    def top_logprobs_prompt(self, slot, k):
        return [(65 + i, -1.0 - i) for i in range(k)]

    def close(self):
        pass


def make_server(reply_text=None, reply=None, **kw):
    """(server, scheduler, engine, prompter); the scheduler thread is started (unless ``start=False``: the test drives the
    scheduler's steps by hand), the watchdog is not."""
    from qwserve.api import Server
    from qwserve.scheduler import Scheduler
    pr = make_prompter()
    if reply is None:
        ids = pr.encode(reply_text if reply_text is not None else "hello world")
        reply = lambda prompt: ids
    eng = FakeEngine(reply, eos=pr.token_id("<|im_end|>"), **{k: v for k, v in kw.items() if k in ("slots", "step_seconds")})
    sched = Scheduler(eng, drafts=kw.get("drafts", 0), prefill_piece=kw.get("piece", 2048), stuck_seconds=kw.get("stuck_seconds", 300.0),
                      log=kw.get("log", lambda *_: None))
    srv = Server(eng, pr, sched, "qw-test", default_budget=kw.get("default_budget", 0))
    if kw.get("start", True):
        sched.start(watchdog=False)
    return srv, sched, eng, pr
