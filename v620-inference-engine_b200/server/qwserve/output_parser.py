"""Token-level router of the model's output into reasoning (<think> ... </think>), tool calls
(<tool_call> ... </tool_call>) and plain content, working on token ids so a tag split over stream chunks is
never emitted as text (reference behaviour: server/qwserve/output_parser.py:11-65)."""
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class TagIds:
    think_open: Optional[int] = None
    think_close: Optional[int] = None
    tool_open: Optional[int] = None
    tool_close: Optional[int] = None


@dataclass
class Routed:
    channel: str          # "reasoning" | "content" | "tool"
    token: int


class OutputParser:
    def __init__(self, tags: TagIds, start_in_think: bool = False):
        self.tags = tags
        self.state = "reasoning" if start_in_think else "content"
        self.tool_tokens: List[List[int]] = []
        self.reasoning_tokens = 0

    def push(self, tok: int) -> Optional[Routed]:
        t = self.tags
        if tok == t.think_open and t.think_open is not None:
            self.state = "reasoning"
            return None
        if tok == t.think_close and t.think_close is not None:
            self.state = "content"
            return None
        if tok == t.tool_open and t.tool_open is not None:
            self.state = "tool"
            self.tool_tokens.append([])
            return None
        if tok == t.tool_close and t.tool_close is not None:
            self.state = "content"
            return None
        if self.state == "tool":
            self.tool_tokens[-1].append(tok)
            return Routed("tool", tok)
        if self.state == "reasoning":
            self.reasoning_tokens += 1
        return Routed(self.state, tok)
