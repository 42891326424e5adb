"""Vision embedding cache, media keys and the slice-to-rank split.

* A media item is identified by its content hash; its tokens enter the language model as negative ids derived
  from that hash, so the prefix cache tells two images apart and recognises the same image in another prompt
  (reference: src/session/vision_cache.cpp:16-33).
* The tower's output is cached per slice (an image, or one temporal patch of a video) under an LRU byte budget;
  only the slices whose tokens are about to be prefilled are encoded (vision_cache.cpp:37-104).
* With several GPUs, whole slices are spread over the ranks longest first (src/engine/vision_job.hip:15-35)."""
from __future__ import annotations

import collections
from typing import Callable, Dict, List, Sequence, Tuple

import torch

MASK63 = (1 << 63) - 1


def _mix(x: int) -> int:          # splitmix64 finaliser
    x &= 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return x ^ (x >> 31)


def media_key(content_hash: int, slice_index: int, token_index: int, video: bool = False) -> int:
    """The (negative, 32-bit) token id of one vision token: a hash of the media's content hash and the token's place in
    it.  Never 0 or positive, so it cannot collide with a text token; the magnitude is odd for image tokens and even
    for video tokens (``ModelConfig.real_token`` reads the pad token to hash and embed from that bit)."""
    v = _mix(content_hash ^ _mix((slice_index << 32) | token_index)) & 0x7FFFFFFE
    v |= 0 if video else 1
    return -(v if v else 2)


def assign_slices(costs: Sequence[float], ranks: int) -> List[List[int]]:
    """Slices to ranks, most expensive first onto the least loaded rank."""
    load = [0.0] * ranks
    out: List[List[int]] = [[] for _ in range(ranks)]
    for i in sorted(range(len(costs)), key=lambda j: -costs[j]):
        r = min(range(ranks), key=lambda q: load[q])
        out[r].append(i)
        load[r] += costs[i]
    return out


def slice_cost(h: int, w: int) -> float:
    """Relative tower time of an h x w slice: linear terms plus the quadratic attention term."""
    L = h * w
    return L * 1.0 + L * L / 6000.0


class VisionCache:
    def __init__(self, encode: Callable[[torch.Tensor, int, int], torch.Tensor], budget_bytes: int = 2 << 30):
        self.encode, self.budget = encode, budget_bytes
        self.lru: "collections.OrderedDict[Tuple[int, int], torch.Tensor]" = collections.OrderedDict()
        self.bytes = 0
        self.hits = self.misses = 0

    def get(self, content_hash: int, slice_index: int, patches, h: int, w: int) -> torch.Tensor:
        k = (content_hash, slice_index)
        t = self.lru.get(k)
        if t is not None:
            self.lru.move_to_end(k)
            self.hits += 1
            return t
        self.misses += 1
        t = self.encode(patches, h, w)
        self.lru[k] = t
        self.bytes += t.numel() * t.element_size()
        while self.bytes > self.budget and len(self.lru) > 1:
            _, old = self.lru.popitem(last=False)
            self.bytes -= old.numel() * old.element_size()
        return t
