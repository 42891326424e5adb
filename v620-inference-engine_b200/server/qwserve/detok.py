"""Incremental detokenisation that never emits half a UTF-8 character: text is released only up to the last
position where decoding the tokens so far does not end in a replacement character."""
from typing import Callable, List


class IncrementalDetok:
    def __init__(self, decode: Callable[[List[int]], str]):
        self.decode = decode
        self.ids: List[int] = []
        self.sent = 0          # characters already released
        self.base = 0          # tokens folded into the stable prefix
        self.prefix = ""

    def push(self, tok: int) -> str:
        self.ids.append(tok)
        text = self.prefix + self.decode(self.ids[self.base:])
        if text.endswith("�"):
            return ""          # an incomplete multi-byte character: wait for the next token
        out = text[self.sent:]
        self.sent = len(text)
        if len(self.ids) - self.base > 64:      # keep the re-decoded window short
            self.prefix, self.base = text, len(self.ids)
        return out

    def flush(self) -> str:
        text = self.prefix + self.decode(self.ids[self.base:])
        out = text[self.sent:]
        self.sent = len(text)
        return out
