"""Glue between the C API's media descriptors, the vision tower and the engine's prefill: media tokens get ids
derived from the content hash, and the rows of a prompt chunk that carry such ids take their embedding from the
tower's (cached) output instead of the embedding table (reference: src/session/vision_cache.cpp:26-104,
src/capi/capi.cpp media entry points)."""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .cache import VisionCache, media_key
from .encoder import VisionEncoder


class VisionFrontend:
    def __init__(self, encoder: VisionEncoder, cache_bytes: int = 2 << 30):
        self.enc = encoder
        self.cache = VisionCache(encoder.encode, cache_bytes)
        self.slices: Dict[Tuple[int, int], Tuple[np.ndarray, int, int]] = {}      # (hash, slice) -> patches, h, w
        self.where: Dict[int, Tuple[int, int, int]] = {}                            # token id -> hash, slice, row

    def add_media(self, tokens: List[int], content_hash: int, video: bool, t: int, h: int, w: int, patches: np.ndarray,
                  starts: Sequence[int]) -> None:
        """Rewrite the media's placeholder positions in ``tokens`` with its ids and keep its patches for encoding."""
        merge = self.enc.cfg.merge
        per, rows = h * w // (merge * merge), h * w
        for sl in range(t):
            self.slices[(content_hash, sl)] = (np.ascontiguousarray(patches[sl * rows:(sl + 1) * rows]), h, w)
            s0 = int(starts[sl])
            if s0 < 0 or s0 + per > len(tokens):
                raise ValueError("a media slice lies outside the prompt")
            for j in range(per):
                k = media_key(content_hash, sl, j, video)
                tokens[s0 + j] = k
                self.where[k] = (content_hash, sl, j)

    def read_media(self, media_addr: int, n_media: int) -> list:
        """The ``n_media`` qw_media structs at ``media_addr`` as plain values (hash, video, t, h, w, patches, starts):
        copies, so that they can travel to the other ranks' processes."""
        from ..capi_impl import QwMedia
        arr = (QwMedia * n_media).from_address(media_addr)
        out = []
        for m in arr:
            rows = m.t * m.h * m.w
            patches = np.ctypeslib.as_array(m.patches, shape=(rows, self.enc.cfg.patch_in)).copy()
            starts = np.ctypeslib.as_array(m.starts, shape=(m.t,)).copy()
            out.append((int(m.hash), bool(m.video), int(m.t), int(m.h), int(m.w), patches, starts))
        return out

    def map_media(self, tokens: List[int], media: list) -> List[int]:
        """Register the media (values of ``read_media``) and return the prompt with its pad tokens replaced by vision ids."""
        out = list(tokens)
        for hsh, video, t, h, w, patches, starts in media:
            self.add_media(out, hsh, video, t, h, w, patches, starts)
        return out

    def map_media_tokens(self, tokens: List[int], media_addr: int, n_media: int) -> List[int]:
        """C API entry: ``media_addr`` points at ``n_media`` qw_media structs."""
        return self.map_media(tokens, self.read_media(media_addr, n_media))

    def stage(self, slot, media_addr, n_media) -> None:
        """Nothing to do ahead of time: slices are encoded when the chunk that holds their tokens is prefilled."""

    def lookup(self, ids: Sequence[int]) -> Optional[torch.Tensor]:
        """Embeddings [len(ids), width] of vision token ids (device, fp32)."""
        rows = []
        for k in ids:
            if k not in self.where:
                raise ValueError(f"vision token {k} belongs to no media of this prompt")
            hsh, sl, j = self.where[k]
            patches, h, w = self.slices[(hsh, sl)]
            rows.append(self.cache.get(hsh, sl, patches, h, w)[j])
        return torch.stack(rows) if rows else None
