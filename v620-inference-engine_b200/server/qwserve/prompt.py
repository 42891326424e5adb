"""Prompt rendering: sandboxed Jinja2 chat template + HF ``tokenizers`` tokenizer, and the mapping of the
various client conventions for "thinking" onto (enabled, effort, budget)
(reference behaviour: server/qwserve/prompt.py:13-134)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Tuple

from jinja2.sandbox import ImmutableSandboxedEnvironment


class Prompter:
    def __init__(self, model_dir: Optional[str] = None, tokenizer=None, template: Optional[str] = None):
        if tokenizer is None:
            from tokenizers import Tokenizer
            tokenizer = Tokenizer.from_file(os.path.join(model_dir, "tokenizer.json"))
        self.tok = tokenizer
        if template is None:
            p = os.path.join(model_dir, "chat_template.jinja")
            if os.path.exists(p):
                template = open(p).read()
            else:
                cfg = json.load(open(os.path.join(model_dir, "tokenizer_config.json")))
                template = cfg["chat_template"]
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False, **{k: w for k, w in kw.items() if k == "indent"})
        env.globals["raise_exception"] = self._raise
        self.template = env.from_string(template)

    @staticmethod
    def _raise(msg):
        raise ValueError(msg)

    def token_id(self, text: str) -> Optional[int]:
        return self.tok.token_to_id(text)

    def render(self, messages: List[dict], tools: Optional[List[dict]] = None, add_generation_prompt: bool = True,
               enable_thinking: bool = True, **kw) -> str:
        return self.template.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                                    enable_thinking=enable_thinking, **kw)

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False).ids

    def encode_batch(self, texts: List[str]) -> List[List[int]]:
        return [e.ids for e in self.tok.encode_batch(texts, add_special_tokens=False)]

    def decode(self, ids: List[int]) -> str:
        return self.tok.decode(ids, skip_special_tokens=False)


EFFORT_BUDGET = {"low": 1024, "medium": 8192, "high": 32768, "xhigh": 0}


def resolve_thinking(body: Dict[str, Any], default_effort: Optional[str] = None,
                     default_budget: int = 0) -> Tuple[bool, Optional[str], int]:
    """(enabled, effort, budget in tokens; 0 = unlimited) from OpenAI (`reasoning_effort`, `reasoning.effort`),
    vLLM (`chat_template_kwargs.enable_thinking`), Anthropic (`thinking: {type, budget_tokens}`) and
    opencode (`thinking_budget`) style fields."""
    enabled, effort, budget = True, default_effort, default_budget
    ctk = body.get("chat_template_kwargs") or {}
    if "enable_thinking" in ctk:
        enabled = bool(ctk["enable_thinking"])
    if "enable_thinking" in body:
        enabled = bool(body["enable_thinking"])
    th = body.get("thinking")
    if isinstance(th, dict):
        if th.get("type") == "disabled":
            enabled = False
        elif th.get("type") == "enabled":
            enabled = True
            if th.get("budget_tokens"):
                budget = int(th["budget_tokens"])
    eff = body.get("reasoning_effort") or (body.get("reasoning") or {}).get("effort")
    if eff:
        eff = str(eff).lower()
        if eff in ("none", "off", "minimal"):
            enabled = False
        else:
            effort = eff
            budget = EFFORT_BUDGET.get(eff, budget)
    if body.get("thinking_budget") is not None:
        budget = int(body["thinking_budget"])
        if budget < 0:
            enabled = False
    return enabled, effort, max(0, budget)
