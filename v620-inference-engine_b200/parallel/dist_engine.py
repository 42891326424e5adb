"""Multi-GPU engine set-up: one process per GPU (torchrun), TP + EP over ``world`` ranks.

Two collective backends for the same engine:

* ``p2p``  – this library's kernel-initiated collectives over NVLink peer memory (``ops/csrc/p2p.cu``):
  a symmetric region is allocated with ``torch.distributed._symmetric_memory`` (which only does the
  allocation and the pointer exchange), and every collective of the decode step is one kernel that
  pushes into the peers' slots and reduces in rank order.  The whole step, including the
  vocabulary-parallel argmax merge, stays on the device, so it can be chained and graph-captured.
* ``nccl`` – the unfused baseline: the runtime calls back into Python at every collective site and
  ``torch.distributed`` (NCCL) does the all-reduce / all-gather / reduce-scatter.

(Reference: the hand-written push collectives of src/comm/comm.hip and the schedule of
src/engine/decode.hip:40-163; there is no NCCL path in the reference.)
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..engine.engine import Engine, EngineOptions
from ..models.config import ModelConfig
from ..ops import structs as S


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class SymmetricRegion:
    """A byte region that exists at the same size on every rank, with every rank's base pointer."""

    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.nbytes = nbytes
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass
        self.tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.tensor.zero_()
        try:
            self.handle = symm_mem.rendezvous(self.tensor, group=group)
        except TypeError:
            self.handle = symm_mem.rendezvous(self.tensor, group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)


def attach_p2p(eng: Engine, group=None) -> None:
    dm = eng.dm
    c, sc, R = dm.cfg, dm.sc, dm.sc.ranks
    rows = dm.max_rows
    lay, off = {}, 0

    def take(name, n):
        nonlocal off
        lay[name] = off
        off = _align(off + n)
    for k in range(4):
        take(f"flags{k}", 2 * R * 64)
    # receive slots hold 8-byte words {payload, sequence number} for the fused collectives (the stand-alone
    # kernels use the first half of a slot for plain fp32)
    slot0 = rows * sc.hc_send * 8
    slot1 = rows * sc.sh * 8
    slot2 = rows * sc.sh * 8
    take("recv0", 2 * R * slot0)
    take("recv1", 2 * R * slot1)
    take("recv2", 2 * R * slot2)
    take("bin", rows * c.hidden * 2)
    take("amax", rows * R * 2 * 4)
    take("mtp_hid", rows * c.hc * c.hidden * 4)
    take("logits", rows * c.vocab * 4)
    region = SymmetricRegion(off, dm.dev, group)
    p = S.QwP2P()
    for i in range(8):
        p.peer[i] = region.ptrs[i] if i < R else None
    p.ranks, p.rank = R, sc.rank
    dm.p2p_base = torch.zeros(1, dtype=torch.int32, device=dm.dev)
    p.base = dm.p2p_base.data_ptr()
    for k in range(4):
        p.off_flags[k] = lay[f"flags{k}"]
    p.off_recv[0], p.slot_bytes[0] = lay["recv0"], slot0
    p.off_recv[2], p.slot_bytes[2] = lay["recv2"], slot2
    p.off_recv[1], p.slot_bytes[1] = lay["recv1"], slot1
    p.off_recv[3] = 0
    p.slot_bytes[3] = 0
    p.off_bin, p.off_amax = lay["bin"], lay["amax"]
    dm.p2p, dm.p2p_region = p, region
    base = region.ptrs[sc.rank]
    # the block-input matrix and the argmax pairs live inside the region (all-gather targets)
    raw = region.tensor
    dm.buf["bin"] = raw[lay["bin"]: lay["bin"] + rows * c.hidden * 2].view(torch.bfloat16).view(rows, c.hidden)
    dm.model.b.bin = base + lay["bin"]
    dm.model.p2p = C.cast(C.pointer(p), C.c_void_p)
    dm.model.amax_pairs = base + lay["amax"]
    dm.model.off_amax = lay["amax"]
    dm.model.off_bin = lay["bin"]
    dm.model.mtp_hid = base + lay["mtp_hid"]
    dm.model.off_mtp_hid = lay["mtp_hid"]
    # the logits buffer becomes this rank's column slice of the [rows][vocab] matrix all ranks' slices are gathered into
    full = raw[lay["logits"]: lay["logits"] + rows * c.vocab * 4].view(torch.float32).view(rows, c.vocab)
    dm.logits_full = full
    dm.buf["logits"] = full[:, sc.rank * sc.vocab_l:(sc.rank + 1) * sc.vocab_l]
    dm.model.b.logits = base + lay["logits"] + sc.rank * sc.vocab_l * 4
    dm.model.off_logits = lay["logits"]
    dm.model.logits_ld = c.vocab
    dm.graphs.clear()


def attach_tp(eng: Engine, group=None, lanes: int = 0) -> None:
    """Channels of the token-major prefill (``ops/csrc/tp.cuh``): one symmetric region per micro-batch lane, sized for
    the engine's prefill chunk.  Without them a multi-rank engine prefills with the row-batched decode kernels."""
    from ..utils import settings
    from . import tp_channel
    dm = eng.dm
    if eng.opts.prefill_chunk <= 0 or dm.sc.ranks == 1:
        return
    # measured per 4,096-token chunk, one lane / two lanes: 132.6 / 142.7 ms on 2 GPUs, 106.9 / 107.1 on 4, 95.9 / 93.2 on 8
    lanes = lanes or settings.get().prefill_lanes or (2 if dm.sc.ranks >= 8 else 1)
    rows = min(eng.opts.prefill_chunk, max(256, dm.slot_tokens))
    eng.tp_channels = [tp_channel.make_symmetric(dm.cfg, dm.sc, rows, dm.dev, bool(dm.cfg.mtp), group) for _ in range(lanes)]
    eng.prefiller = None


def set_fused(on: bool) -> None:
    """Peer-memory backend: send every collective from the kernel that produces its payload and wait for it in
    the kernel that consumes it (default), or run each collective as a kernel of its own."""
    from ..ops import lib as qlib
    qlib.load(True).qwrt_set_fuse(int(on))


def attach_nccl(eng: Engine, group=None) -> None:
    """Unfused baseline: NCCL collectives through torch.distributed at every site."""
    dm = eng.dm
    group = group or dist.group.WORLD
    R, sc, c = dm.sc.ranks, dm.sc, dm.cfg
    b = dm.buf
    ptr2buf = {b[n].data_ptr(): b[n] for n in ("send", "red", "ple_send", "ple_red", "partial", "out_a", "out_b", "bin")}

    def cb(user, kind, site, src, dst, rows, n, stream):
        if kind == 0:
            s, d = ptr2buf[src], ptr2buf[dst]
            d[:rows].copy_(s[:rows])
            dist.all_reduce(d[:rows], group=group)
        elif kind == 1:
            bin_ = b["bin"]
            mine = bin_[:rows, sc.rank * n:(sc.rank + 1) * n].contiguous()
            out = torch.empty((R, rows, n), dtype=bin_.dtype, device=bin_.device)
            dist.all_gather_into_tensor(out, mine, group=group)
            bin_[:rows].copy_(out.permute(1, 0, 2).reshape(rows, R * n))
        else:
            s, d = ptr2buf[src], ptr2buf[dst]
            inp = s[:rows].view(rows, R, n).permute(1, 0, 2).contiguous()
            dist.reduce_scatter_tensor(d[:rows], inp, group=group)

    dm.set_comm(cb)
    dm.model.p2p = None
    dm.model.mtp.enabled = 0             # the MTP pass gathers hidden states through the peer-memory backend only
    eng.opts.use_graphs = False          # the collectives are enqueued from a host callback: steps are not graph-captured

    def merge_argmax(M):
        val, idx = b["amax_val"][:M].contiguous(), b["amax_idx"][:M].contiguous()
        vs = torch.empty((R, M), dtype=val.dtype, device=val.device)
        ix = torch.empty((R, M), dtype=idx.dtype, device=idx.device)
        dist.all_gather_into_tensor(vs, val, group=group)
        dist.all_gather_into_tensor(ix, idx, group=group)
        best = vs.max(0).values
        cand = torch.where(vs == best, ix, torch.full_like(ix, 2**31 - 1))
        b["amax_idx"][:M].copy_(cand.min(0).values)
        b["amax_val"][:M].copy_(best)
    eng.merge_argmax = merge_argmax
    dm.graphs.clear()


def make_engine(cfg: ModelConfig, opts: EngineOptions, world: int, rank: int, device: str, ple_rows: int = 1 << 20,
                log: Optional[Callable[[str], None]] = None, comm: str = "p2p", seed: int = 0,
                exact: bool = False) -> Engine:
    """Build this rank's engine with random-init weights of ``cfg`` and attach the collectives."""
    eng = Engine.synthetic(cfg, opts, ranks=world, rank=rank, device=device, seed=seed, exact=exact,
                           ple_rows=ple_rows, log=log)
    if world > 1:
        if comm in ("p2p", "p2p-unfused"):
            attach_p2p(eng)
            set_fused(comm == "p2p")
            attach_tp(eng)
        else:
            attach_nccl(eng)
    return eng
