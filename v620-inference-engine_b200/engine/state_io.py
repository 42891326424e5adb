"""Slot state export / import: KV pages for the prefix cache's blocks, recurrent state for snapshots,
VRAM snapshots and slot copies.

A KV block = one page (256 tokens) of every QSA layer; its payload per rank is, layer by layer,
``K[n][row] bf16 | V[n][row] bf16 | ck[n/4][128] bf16`` — the reference's block payload
(src/engine/host_tier.hip:23-30,78-90) with bf16 where it stores fp16.  The recurrent payload is
``GDN S | GDN conv ring | PLE ring | raw-key ring`` in fp32 (host_tier.hip:121-137).  A saved state is
valid only for the same ``state_layout_id`` (host_tier.hip:269-281): an FNV-1a hash of a version and
every shape that enters the payloads.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from .device_model import DeviceModel, KV_PAGE

LAYOUT_VERSION = 1


def _fnv(vals) -> int:
    h = 0xcbf29ce484222325
    for v in vals:
        for b in int(v).to_bytes(8, "little", signed=False):
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


class StateIO:
    def __init__(self, dm: DeviceModel):
        self.dm = dm
        c, sc = dm.cfg, dm.sc
        self.row = sc.kvh_l * c.head_dim
        self.groups = KV_PAGE // c.idx_ratio
        self.kv_page_elems = 2 * KV_PAGE * self.row + self.groups * c.idx_dim      # per layer, bf16 elements
        self.kv_block_bytes = len(dm.k_dev) * self.kv_page_elems * 2

    def state_layout_id(self) -> int:
        c, sc = self.dm.cfg, self.dm.sc
        return _fnv([LAYOUT_VERSION, sc.ranks, c.n_layers, c.n_qsa, c.n_gdn, self.row, c.idx_dim, c.idx_ratio, KV_PAGE,
                     sc.gdn_vl, c.gdn_dim, sc.gdn_qkv_l, sc.xw, self.dm.gdn_ring[0].shape[1] if c.n_gdn else 0,
                     self.dm.ple_ring.shape[1], self.dm.raw_ring[0].shape[1] if c.n_qsa else 0])

    # ---- KV pages
    def _page_views(self, slot: int, page_index: int):
        dm = self.dm
        pid = int(dm.page_table_host[slot, page_index])
        out = []
        for qi in range(len(dm.k_dev)):            # QSA layers, then the MTP layer's own cache
            if pid < dm.n_dev_pages:
                k, v = dm.k_dev[qi][pid], dm.v_dev[qi][pid]
            else:
                k, v = dm.k_host[qi][pid - dm.n_dev_pages], dm.v_host[qi][pid - dm.n_dev_pages]
            ck = dm.ck[qi][slot, page_index * self.groups:(page_index + 1) * self.groups]
            out.append((k, v, ck))
        return out

    def export_kv(self, slot: int, page_index: int) -> bytes:
        parts = []
        for k, v, ck in self._page_views(slot, page_index):
            parts += [k.reshape(-1).to(self.dm.dev), v.reshape(-1).to(self.dm.dev), ck.reshape(-1)]
        return torch.cat(parts).view(torch.int16).cpu().numpy().tobytes()

    def import_kv(self, slot: int, page_index: int, payload: bytes) -> None:
        assert len(payload) == self.kv_block_bytes, "KV block size does not match this engine's layout"
        t = torch.from_numpy(np.frombuffer(payload, dtype=np.int16).copy()).view(torch.bfloat16)
        off = 0
        for k, v, ck in self._page_views(slot, page_index):
            for dst in (k, v, ck):
                n = dst.numel()
                dst.copy_(t[off:off + n].view(dst.shape).to(dst.device))
                off += n
        self.dm.spill_cache_clear()         # the page may live in host memory: cached copies of its rows are stale now

    # ---- KV pages through pinned units: one gather launch + one asynchronous copy per block
    MAX_BATCH = 8          # blocks moved per call (a 2,048-token prefill piece)

    def _ensure_staging(self):
        if getattr(self, "stage", None) is not None:
            return
        dm = self.dm
        nseg = self.MAX_BATCH * 3 * len(dm.k_dev)
        self.stage = torch.zeros(self.MAX_BATCH * self.kv_block_bytes, dtype=torch.uint8, device=dm.dev)
        self.tab_host = torch.zeros(3 * nseg, dtype=torch.int64).pin_memory()       # src | dst | bytes
        self.tab_dev = torch.zeros(3 * nseg, dtype=torch.int64, device=dm.dev)
        self.nseg_max = nseg

    def _segments(self, slot: int, page_indices, to_stage: bool):
        """Fill the segment tables for moving the given pages between the slot state and the staging buffer."""
        import ctypes as C
        self._ensure_staging()
        assert len(page_indices) <= self.MAX_BATCH
        if getattr(self, "tab_event", None) is not None:
            self.tab_event.synchronize()          # the previous call's copy of the tables has run
        tab = self.tab_host.numpy()
        n, base = 0, self.stage.data_ptr()
        for b, pi in enumerate(page_indices):
            off = b * self.kv_block_bytes
            for k, v, ck in self._page_views(slot, pi):
                for t in (k, v, ck):
                    nb = t.numel() * 2
                    state, st = t.data_ptr(), base + off
                    tab[n], tab[self.nseg_max + n], tab[2 * self.nseg_max + n] = (state, st, nb) if to_stage else (st, state, nb)
                    off += nb
                    n += 1
        self.tab_dev.copy_(self.tab_host, non_blocking=True)
        self.tab_event = torch.cuda.Event()
        self.tab_event.record(torch.cuda.current_stream(self.dm.dev))
        s = C.c_void_p(torch.cuda.current_stream(self.dm.dev).cuda_stream)
        p = self.tab_dev.data_ptr()
        return n, C.c_void_p(p), C.c_void_p(p + 8 * self.nseg_max), C.c_void_p(p + 16 * self.nseg_max), s

    def export_kv_units(self, slot: int, page_indices, units) -> None:
        """Enqueue the export of the given pages, block i into ``units[i]`` (uint8 arrays over pinned host memory of at
        least ``kv_block_bytes``).  Asynchronous: ``sync()`` before the units are read."""
        import ctypes as C
        n, src, dst, nb, s = self._segments(slot, page_indices, True)
        L = self.dm.lib
        if L.qwk_segments_copy(src, dst, nb, n, s) != 0:
            raise RuntimeError("qwk_segments_copy failed")
        for b, u in enumerate(units):
            if L.qwk_memcpy_async(C.c_void_p(u.ctypes.data), C.c_void_p(self.stage.data_ptr() + b * self.kv_block_bytes),
                                  self.kv_block_bytes, 2, s) != 0:
                raise RuntimeError("qwk_memcpy_async failed")

    def import_kv_units(self, slot: int, page_indices, units) -> None:
        """The reverse: ``units[i]`` holds the payload of page ``page_indices[i]``.  Asynchronous on the current stream (the
        units must stay untouched until ``sync()``)."""
        import ctypes as C
        L = self.dm.lib
        s = C.c_void_p(torch.cuda.current_stream(self.dm.dev).cuda_stream)
        self._ensure_staging()
        for b, u in enumerate(units):
            if L.qwk_memcpy_async(C.c_void_p(self.stage.data_ptr() + b * self.kv_block_bytes), C.c_void_p(u.ctypes.data),
                                  self.kv_block_bytes, 1, s) != 0:
                raise RuntimeError("qwk_memcpy_async failed")
        n, src, dst, nb, s = self._segments(slot, page_indices, False)
        if L.qwk_segments_copy(src, dst, nb, n, s) != 0:
            raise RuntimeError("qwk_segments_copy failed")
        self.dm.spill_cache_clear()

    def sync(self) -> None:
        torch.cuda.current_stream(self.dm.dev).synchronize()

    # ---- recurrent state
    def _recurrent_tensors(self, slot: int) -> List[torch.Tensor]:
        dm = self.dm
        ts = [t[slot] for t in dm.gdn_S] + [t[slot] for t in dm.gdn_ring] + [dm.ple_ring[slot]] + [t[slot] for t in dm.raw_ring]
        return ts

    def recurrent_bytes(self) -> int:
        return sum(t.numel() * 4 for t in self._recurrent_tensors(0))

    def _recurrent_pinned(self) -> torch.Tensor:
        """One pinned buffer of ``recurrent_bytes`` for snapshots on their way to and from the host store."""
        if getattr(self, "_rec_pin", None) is None:
            self._rec_pin = torch.empty(self.recurrent_bytes(), dtype=torch.uint8).pin_memory()
        return self._rec_pin

    def export_recurrent_pinned(self, slot: int):
        """The slot's recurrent state in the pinned snapshot buffer (asynchronous copies, then one wait).  Returns
        (address, bytes); the buffer is reused by the next export or import."""
        pin = self._recurrent_pinned().view(torch.float32)
        off = 0
        for t in self._recurrent_tensors(slot):
            n = t.numel()
            pin[off:off + n].view(t.shape).copy_(t, non_blocking=True)
            off += n
        self.sync()
        return pin.data_ptr(), off * 4

    def import_recurrent_pinned(self, slot: int) -> None:
        """The reverse: the pinned snapshot buffer (filled by the caller) becomes the slot's recurrent state."""
        pin = self._recurrent_pinned().view(torch.float32)
        off = 0
        for dst in self._recurrent_tensors(slot):
            n = dst.numel()
            dst.copy_(pin[off:off + n].view(dst.shape), non_blocking=True)
            off += n
        self.sync()

    def export_recurrent(self, slot: int) -> bytes:
        return torch.cat([t.reshape(-1) for t in self._recurrent_tensors(slot)]).cpu().numpy().tobytes()

    def import_recurrent(self, slot: int, payload: bytes) -> None:
        t = torch.from_numpy(np.frombuffer(payload, dtype=np.float32).copy()).to(self.dm.dev)
        off = 0
        for dst in self._recurrent_tensors(slot):
            n = dst.numel()
            dst.copy_(t[off:off + n].view(dst.shape))
            off += n
        assert off == t.numel(), "recurrent payload size does not match this engine's layout"

    # ---- VRAM snapshots / slot copy
    def snapshot_save(self, slot: int):
        """Recurrent state kept on the device (cheap: no host round trip)."""
        return [t.clone() for t in self._recurrent_tensors(slot)]

    def snapshot_restore(self, slot: int, snap) -> None:
        for dst, src in zip(self._recurrent_tensors(slot), snap):
            dst.copy_(src)

    def slot_copy(self, src: int, dst: int, n_tokens: int) -> None:
        """Make ``dst`` hold the first ``n_tokens`` of ``src`` (whole pages of KV + the recurrent state as it
        is now: the caller copies at a point where the state matches ``n_tokens``)."""
        dm = self.dm
        pages = (n_tokens + KV_PAGE - 1) // KV_PAGE
        for p in range(pages):
            for (ks, vs, cs), (kd, vd, cd) in zip(self._page_views(src, p), self._page_views(dst, p)):
                kd.copy_(ks)
                vd.copy_(vs)
                cd.copy_(cs)
        dm.spill_cache_clear()
        for d, s in zip(self._recurrent_tensors(dst), self._recurrent_tensors(src)):
            d.copy_(s)
