"""Non-prefix reuse of a cached chunk (the CacheBlend-style experiment): the mathematics, kept as an experiment.

A prefix cache can only reuse a prompt's leading tokens, because the GDN state after a chunk depends on everything
before the chunk.  The delta rule is, however, *affine* in the state that enters it,

    S_out = M S_in + U,      M = prod_t  exp(g_t) (I - beta_t k_t k_t^T)      (per value head, dim x dim),

so a chunk recorded once (S_in, S_out and M) can be re-based onto another prefix's state S with
``S_out + M (S - S_in)``; the chunk's K rows are re-rotated to their new positions and the position-indexed rings
are moved by the position shift.  The reference built this (src/kernels/blend.hpp:14-25,
src/engine/blend.hip:18-93), measured it and rejected it: the composition is exact only for layers whose inputs do
not depend on the context (layer 0); deeper layers' activations change with the prefix and nothing corrects that
(its docs/DESIGN.md:183-224).  Its splice step refuses to run since the slots keep only a ring of raw indexer keys.
Nothing in serving calls this module; ``Session`` only counts how many prompt tokens such reuse could have covered
(``blend_candidate_tokens``).

Design: M needs no kernel of its own.  The columns of S evolve independently under the recurrence, so M is what
the ordinary scan produces from the initial state I with every v_t = 0; any scan with the signature of
``delta_scan`` will do (the engine's chunked prefill kernel ``qwk_gdn_scan_chunked`` computes the same recurrence
from post-convolution q, k, v, decay and beta).  The composition is one batched 128 x 128 x 128 product per layer.
Everything here is plain PyTorch on whatever device the tensors live on; it is not a hot path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..models.config import ModelConfig
from ..models.reference import rope


def delta_scan(S: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """The gated delta rule over T tokens, fp32.  S [heads][dim k][dim v] (returned, not modified); k, v
    [T][heads][dim]; g (log decay) and beta [T][heads].  Same recurrence as ``RefModel.gdn``."""
    S = S.float().clone()
    for t in range(k.shape[0]):
        S = S * torch.exp(g[t]).view(-1, 1, 1)
        u = (v[t] - torch.einsum("hkv,hk->hv", S, k[t])) * beta[t].unsqueeze(-1)
        S = S + k[t].unsqueeze(-1) * u.unsqueeze(1)
    return S


Scan = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


def transfer_init(heads: int, dim: int, device=None) -> torch.Tensor:
    """M of an empty chunk: the identity for every head."""
    return torch.eye(dim, dtype=torch.float32, device=device).repeat(heads, 1, 1)


def transfer_advance(M: torch.Tensor, k: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, scan: Scan = delta_scan) -> torch.Tensor:
    """M after T more tokens (called once per prefill piece of the chunk being recorded): the scan with v = 0,
    started from M.  (Role of the reference's gdn_transfer_T, src/kernels/blend.hip:8-40.)"""
    return scan(M, k, torch.zeros_like(k), g, beta)


def compose(S: torch.Tensor, M: torch.Tensor, S_in: torch.Tensor, S_out: torch.Tensor) -> torch.Tensor:
    """State after the recorded chunk when it follows a prefix that left ``S`` instead of ``S_in``.
    All [heads][dim][dim] (or [layers][heads][dim][dim]).  (src/kernels/blend.hip:57-73.)"""
    return S_out + torch.matmul(M, S - S_in)


def rope_shift(cfg: ModelConfig, K: torch.Tensor, delta: int) -> torch.Tensor:
    """Cached (normed and rotated) keys K [n][..., head_dim] moved by ``delta`` positions: rotations compose, so
    the rotary part is rotated once more by the angle of ``delta``.  (src/kernels/blend.hip:75-86.)"""
    pos = torch.full((K.shape[0],), int(delta), dtype=torch.int64)
    return rope(cfg, K.float(), pos).to(K.dtype)


def ring_cell(cell: int, delta: int, ring: int) -> int:
    """Where the content of a position-indexed ring's ``cell`` lives after the positions moved by ``delta``."""
    return ((cell + delta) % ring + ring) % ring


def shift_ring(ring: torch.Tensor, delta: int, dim: int = 0) -> torch.Tensor:
    """A ring whose cell index is position % size (the GDN convolution ring, the PLE ring), re-indexed for
    positions moved by ``delta`` (src/engine/blend.hip:64-78)."""
    return torch.roll(ring, shifts=int(delta) % ring.shape[dim], dims=dim)


@dataclass
class ChunkRecord:
    """What recording a chunk keeps per GDN layer stack: the states on both sides and the transfer."""
    S_in: torch.Tensor       # [layers][heads][dim][dim], state before the chunk's first token
    S_out: torch.Tensor      # state after its last token
    M: torch.Tensor          # transfer over the chunk
    start: int               # position of the chunk's first token when it was recorded
    length: int

    def rebase(self, S: torch.Tensor, with_transfer: bool = True) -> torch.Tensor:
        """The state after the chunk on top of another prefix's state ``S``.  Without the transfer the recorded
        end state is used as it is (the reference's "no correction" arm)."""
        return compose(S, self.M, self.S_in, self.S_out) if with_transfer else self.S_out.clone()

    def shift(self, new_start: int) -> int:
        return int(new_start) - self.start


def relative_error(a: torch.Tensor, b: torch.Tensor) -> float:
    """|a - b| / |b| over everything: the figure the experiment reports per layer."""
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def record(S_in: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, start: int,
           scan: Scan = delta_scan, M: Optional[torch.Tensor] = None) -> ChunkRecord:
    """Scan one layer's chunk from ``S_in`` and record it (single layer: tensors without the layer axis)."""
    M0 = transfer_init(S_in.shape[0], S_in.shape[1], S_in.device) if M is None else M
    return ChunkRecord(S_in=S_in.float().clone(), S_out=scan(S_in, k, v, g, beta), M=transfer_advance(M0, k, g, beta, scan),
                       start=int(start), length=int(k.shape[0]))
