"""Channels of the tensor-parallel token-major prefill (``ops/csrc/tp.cuh``).

A channel is one region per rank with the same layout - flags, and one receive buffer per collective
kind - plus every rank's base pointer.  The kernels of a prefill chunk store into the peers' regions and
poll their own; this module only lays the region out, allocates it (as symmetric memory across the
processes of a node, or as plain tensors of one process when several ranks are emulated on one GPU for
tests) and fills the ``QwTp`` struct the launchers take.

(Role of the reference's two ``Comm`` instances, one per prefill micro-batch: src/engine/engine.hip:42-44,
src/comm/comm.hip:217-239.)
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch

from ..models.config import ModelConfig, ShardConfig
from ..ops import structs as S


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def layout(cfg: ModelConfig, sc: ShardConfig, rows: int, mtp: bool) -> Dict[str, object]:
    """Byte layout of a region that serves chunks of up to ``rows`` rows."""
    R = sc.ranks
    hc_ld = (cfg.hc_down + 7) // 8 * 8
    part = [0] * S.TP_KINDS
    whole = [0] * S.TP_KINDS
    part[S.TP_SSQ] = _align(rows * cfg.hc * 4)
    part[S.TP_DOWN] = _align(rows * hc_ld * 4)
    part[S.TP_RS] = _align(rows * sc.sh * 4)
    part[S.TP_SMALL] = _align(max(rows * 64, 4096))
    for k in (S.TP_SSQ, S.TP_DOWN, S.TP_RS, S.TP_SMALL):
        whole[k] = R * part[k]
    part[S.TP_BIN] = whole[S.TP_BIN] = _align(rows * cfg.hidden * 2)
    part[S.TP_WIDE] = whole[S.TP_WIDE] = _align(rows * cfg.hc * cfg.hidden * 2) if mtp else 256
    off = _align(S.TP_KINDS * 8 * 64)
    offs = []
    for k in range(S.TP_KINDS):
        offs.append(off)
        off += whole[k]
    return {"off_flags": 0, "off_buf": offs, "part_bytes": part, "nbytes": off, "hc_ld": hc_ld}


class TpChannel:
    """One rank's view of a channel: the filled ``QwTp`` struct and the tensors that keep its memory alive."""

    def __init__(self, lay: Dict[str, object], ranks: int, rank: int, peers: List[int], region: torch.Tensor, device,
                 spin_limit: int = 0):
        self.lay, self.region = lay, region
        self.ticket = torch.zeros(S.TP_KINDS, dtype=torch.int32, device=device)
        t = S.QwTp()
        for i in range(8):
            t.peer[i] = peers[i] if i < ranks else None
        t.ranks, t.rank = ranks, rank
        t.off_flags = lay["off_flags"]
        for k in range(S.TP_KINDS):
            t.off_buf[k] = lay["off_buf"][k]
            t.part_bytes[k] = lay["part_bytes"][k]
            t.seq[k] = 0
        t.ticket = self.ticket.data_ptr()
        t.spin_limit = spin_limit
        self.struct = t
        self.ptr = C.cast(C.pointer(t), C.c_void_p)

    def view(self, kind: int, nbytes: int, dtype=torch.uint8) -> torch.Tensor:
        """This rank's receive buffer of ``kind`` (the first ``nbytes`` bytes) as a tensor."""
        o = self.lay["off_buf"][kind]
        return self.region[o:o + nbytes].view(dtype)

    def set_spin_limit(self, polls: int) -> None:
        self.struct.spin_limit = int(polls)


def make_emulated(cfg: ModelConfig, ranks: int, rows: int, device, mtp: bool, spin_limit: int = 1 << 12) -> List[TpChannel]:
    """The channels of ``ranks`` emulated ranks that live in this process on one device: plain tensors as regions.
    Waits are short (the data is always complete before a consumer runs, see ``qwrt_prefill``)."""
    lays = [layout(cfg, ShardConfig(cfg, ranks, r), rows, mtp) for r in range(ranks)]
    regions = [torch.zeros(lays[r]["nbytes"], dtype=torch.uint8, device=device) for r in range(ranks)]
    peers = [int(t.data_ptr()) for t in regions]
    return [TpChannel(lays[r], ranks, r, peers, regions[r], device, spin_limit) for r in range(ranks)]


def make_symmetric(cfg: ModelConfig, sc: ShardConfig, rows: int, device, mtp: bool, group=None) -> TpChannel:
    """This process's channel over the ranks of ``group`` (one process per GPU): a symmetric-memory region."""
    from .dist_engine import SymmetricRegion
    lay = layout(cfg, sc, rows, mtp)
    reg = SymmetricRegion(lay["nbytes"], device, group)
    ch = TpChannel(lay, sc.ranks, sc.rank, reg.ptrs, reg.tensor, device)
    ch.symm = reg
    return ch
