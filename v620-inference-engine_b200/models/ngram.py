"""N-gram row ids of the PLE table.

For every token position the table is read at ``ngram_heads`` rows: ``ngram-1`` n-gram
orders (2-grams, 3-grams) times ``heads_per_order`` hash heads.  The hash mixes the current
token with its one or two predecessors (replaced by EOS when they lie before the start of the
sequence or before the most recent EOS), multiplies each by an odd 64-bit constant derived
from splitmix64, XORs them and reduces modulo a per-head prime table size
(reference: src/core/ple.cpp:66-125; docs/MODEL.md:192-204).
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

from .config import ModelConfig

MASK = (1 << 64) - 1
GAMMA = 0x9E3779B97F4A7C15


def splitmix64(v: int) -> int:
    v = (v + GAMMA) & MASK
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & MASK
    return (v ^ (v >> 31)) & MASK


_SMALL = (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37)
_WITNESS = (2, 325, 9375, 28178, 450775, 9780504, 1795265022)


def is_prime(n: int) -> bool:
    """Deterministic Miller-Rabin for 64-bit inputs."""
    if n < 2:
        return False
    for p in _SMALL:
        if n % p == 0:
            return n == p
    d, s = n - 1, 0
    while d % 2 == 0:
        d //= 2
        s += 1
    for a in _WITNESS:
        if a % n == 0:
            continue
        x = pow(a, d, n)
        if x in (1, n - 1):
            continue
        for _ in range(s - 1):
            x = pow(x, 2, n)
            if x == n - 1:
                break
        else:
            return False
    return True


class NgramHasher:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        max_mult = ((1 << 63) - 1) // cfg.vocab
        half = max(1, max_mult // 2)
        base_seed = cfg.ple_seed + 10007 * 0      # dense PLE layer id 0
        self.mult = [2 * (splitmix64((base_seed + GAMMA * (i + 1)) & MASK) % half) + 1 for i in range(cfg.ngram)]
        self.sizes: List[int] = []
        self.offsets: List[int] = []
        p, off = cfg.ngram_vocab_base - 1, 0
        for _ in range(cfg.ngram_heads):
            c = p + 1
            if c <= 2:
                c = 2
            else:
                if c % 2 == 0:
                    c += 1
                while not is_prime(c):
                    c += 2
            p = c
            self.sizes.append(p)
            self.offsets.append(off)
            off += p
        self.total_rows = off
        self.per_order = cfg.ngram_heads // (cfg.ngram - 1)

    def ids_for(self, history: Sequence[int], tokens: Sequence[int]) -> np.ndarray:
        """Row ids ``[len(tokens), ngram_heads]`` (int64).  ``history`` is the sequence before
        ``tokens``; only its last ``ngram-1`` entries matter."""
        cfg = self.cfg
        hist = [cfg.real_token(int(t)) for t in list(history)[-(cfg.ngram - 1):]] if len(history) else []
        toks = [cfg.real_token(int(t)) for t in tokens]
        ctx = np.array(hist + toks, dtype=np.int64)
        n_hist, T = len(hist), len(toks)
        out = np.zeros((T, cfg.ngram_heads), dtype=np.int64)
        if T == 0:
            return out
        pos = np.arange(n_hist, n_hist + T)
        # index of the latest EOS strictly before each position (-1 when none)
        is_eos = ctx == cfg.eos
        last = np.where(is_eos, np.arange(len(ctx)), -1)
        last = np.maximum.accumulate(last)
        prev_eos = np.concatenate([[-1], last[:-1]])[pos]
        tok = []
        for s in range(cfg.ngram):
            idx = pos - s
            valid = (idx >= 0) & (idx > prev_eos) if s else np.ones(T, dtype=bool)
            v = np.where(valid, ctx[np.clip(idx, 0, None)], cfg.eos).astype(np.uint64)
            tok.append(v)
        with np.errstate(over="ignore"):
            for order in range(2, cfg.ngram + 1):
                mixed = tok[0] * np.uint64(self.mult[0])
                for i in range(1, order):
                    mixed = mixed ^ (tok[i] * np.uint64(self.mult[i]))
                for j in range(self.per_order):
                    h = (order - 2) * self.per_order + j
                    out[:, h] = (mixed % np.uint64(self.sizes[h])).astype(np.int64) + self.offsets[h]
        return out
