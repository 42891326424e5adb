"""Session: slot bookkeeping and choice, the prefix cache (native block store + disk tier over the engine's
state export / import), sampling, and the speculative generation loop with adaptive draft counts.

This is the layer the C API exposes (reference: ``class Session``, src/session/session.hpp:37-237,
session.cpp, prefix_cache.cpp, generate.cpp).  What is kept from the reference's behaviour:

* ``acquire`` picks the free slot that can reuse the most of the prompt (then least recently used);
* ``begin_prompt`` decides between continuing in place, restoring from the block store (KV blocks up to the
  deepest snapshot on the prompt's path) and resetting;
* prefill runs in pieces so other slots can decode in between, saves a KV block per 256 tokens and a
  snapshot at the end of every piece (pieces end on block boundaries), anchoring message boundaries;
* ``generate`` emits 1..k+1 tokens per request per step: drafts from the MTP head, one verification pass,
  exact sampling per row, accept / rollback, acceptance EMA, and K chosen to maximise expected tokens per
  step cost (1+a+..+a^K)/(base + beta (K-1)).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..engine.engine import Engine
from ..engine.sampling import GpuSampler, SamplingParams
from ..engine.state_io import StateIO
from ..native import host as H

BLOCK = 256
SPEC_BASE, SPEC_BETA = 1.25, 0.25
# Drafting that does not pay (the acceptance average says a step with drafts emits fewer tokens per unit of time than a
# plain one) is switched off for a stretch of steps, then tried again from a probing acceptance; stretches that follow
# one another without a good spell in between grow (reference: plain_step, src/session/generate.cpp:49-86).
PLAIN_FIRST, PLAIN_GROW, PLAIN_MAX, PROBE_ACCEPT, MISSED_MAX = 32, 48, 176, 0.3, 256
VRAM_SNAPSHOTS = 8          # recurrent-state snapshots kept on the device, least recently used first out


@dataclass
class VramSnap:
    """The recurrent state of a slot as it was after its first ``n`` tokens, kept on the device.  The slot's KV rows of
    those tokens stay where they are, so going back to the snapshot costs a few device copies (reference: the snapshot
    table of src/session/session.cpp:37-54 and src/engine/snapshot.hip:19-71)."""
    slot: int
    n: int
    tensors: list
    mtp_hidden: Optional[torch.Tensor]
    logits: Optional[torch.Tensor]
    used: int = 0


@dataclass
class SlotInfo:
    busy: bool = False
    used: int = 0
    prompt: List[int] = field(default_factory=list)      # the whole prompt of the current request
    prompt_end: int = 0
    stop: List[int] = field(default_factory=list)
    logits: Optional[torch.Tensor] = None                 # logits after the prompt (device)
    drafts: List[int] = field(default_factory=list)
    drafts_for: int = -1
    block_keys: List[int] = field(default_factory=list)   # store keys of the slot's full blocks, in order
    last_capture: int = 0                                 # position of the newest device snapshot taken during this prompt
    # running draft acceptance, steps left of a stretch without drafts, length of the next stretch (32 -> 80 -> 128 -> 176):
    # kept by the native planner; ``accept`` / ``plain_left`` / ``plain_stretch`` below read and write its memory
    spec: H.SpecSlot = field(default_factory=lambda: H.SpecSlot(0.5, 0, PLAIN_FIRST), repr=False)
    spec_owner: object = field(default=None, repr=False)
    missed: list = field(default_factory=list)            # MTP rows skipped during the stretch: (hidden, next token, position)
    timing: Dict[str, float] = field(default_factory=lambda: {"restore_s": 0.0, "prefill_s": 0.0, "save_s": 0.0, "pin_wait_s": 0.0})


def _spec_field(name):
    return property(lambda self: getattr(self.spec, name), lambda self, v: setattr(self.spec, name, v))


SlotInfo.accept = _spec_field("accept")
SlotInfo.plain_left = _spec_field("plain_left")
SlotInfo.plain_stretch = _spec_field("plain_stretch")


@dataclass
class StepReq:
    slot: int
    pending: int
    budget: int
    flags: int = 0
    sampling: SamplingParams = field(default_factory=SamplingParams)


@dataclass
class StepOut:
    tokens: List[int]
    logprobs: List[float]
    first_row: int
    stopped: bool


def common_prefix(a: Sequence[int], b: Sequence[int], block: int = 4096) -> int:
    """Length of the longest common prefix.  Whole blocks are compared as list slices (one C-level comparison each), only
    the block that differs is walked token by token: a 131,072-token history costs about a millisecond instead of six."""
    n = min(len(a), len(b))
    if not isinstance(a, list):
        a = list(a)
    if not isinstance(b, list):
        b = list(b)
    i = 0
    while i < n:
        j = min(n, i + block)
        if a[i:j] != b[i:j]:
            while a[i] == b[i]:
                i += 1
            return i
        i = j
    return n


class Session:
    def __init__(self, engine: Engine, host_cache_bytes: int = 8 << 30, disk_cache_dir: Optional[str] = None,
                 disk_cache_bytes: int = 0, prefill_piece: int = 2048, seed: int = 0):
        self.e = engine
        self.cfg = engine.cfg
        from ..utils import settings as _settings
        from ..utils.trace import PhaseTrace
        self.gen_trace = PhaseTrace(_settings.get().trace, "generate")     # QW_TRACE: per-phase milliseconds of generate()
        self.spec_log = bool(_settings.get().spec_log)                     # QW_SPEC_LOG: one line per speculative step and request
        self.spec_max_rows = int(_settings.get().spec_max_rows)            # QW_SPEC_MAX_ROWS: longest verification run of a request (0 = the engine's limit)
        self.io = StateIO(engine.dm)
        n = engine.opts.slots
        self.slots = [SlotInfo() for _ in range(n)]
        # how many drafts, stretches without drafts, what is kept of a verified run: decided natively (native/src/spec_planner.hpp)
        self.planner = H.SpecPlanner(n, SPEC_BASE, SPEC_BETA, PROBE_ACCEPT, PLAIN_FIRST, PLAIN_GROW, PLAIN_MAX)
        for i, si in enumerate(self.slots):
            si.spec = self.planner.slots[i]
            si.spec_owner = self.planner          # the struct lives in the planner's memory: keep it alive as long as the slot record
        self.clock = 0
        self.boundary = -1
        self.piece = max(BLOCK, prefill_piece // BLOCK * BLOCK)
        self.store = H.BlockStore(self.io.state_layout_id(), engine.dm.sc.ranks, host_cache_bytes, disk_cache_dir, disk_cache_bytes)
        self.store_on = host_cache_bytes > 0 or bool(disk_cache_dir)          # no tier to keep blocks in: nothing is exported
        # pinned units for the blocks on their way between the engine and the store (one block per unit)
        self.pool = None
        if torch.cuda.is_available() and (host_cache_bytes > 0 or bool(disk_cache_dir)):          # no store tier: nothing to stage, nothing to pin
            try:
                # QW_POOL_RESERVE_GB: pinned units kept ready for a burst of saves (0: two units; pinning more happens in the
                # background and can stall the host's launches while it runs)
                standing = max(2, int(_settings.get().pool_reserve_gb * (1 << 30)) // max(1, self.io.kv_block_bytes))
                self.pool = H.PinnedPool(self.io.kv_block_bytes, arena_bytes=max(64 << 20, 16 * self.io.kv_block_bytes), standing_units=standing,
                                         use_cuda=True)
            except Exception:
                self.pool = None          # no pinned memory to be had: blocks take the pageable path
        self.sampler = GpuSampler(engine.dm.lib, engine.dm.dev, engine.cfg.vocab, n, engine.opts.max_rows, seed)
        self.sampler.host_only = not _settings.get().gpu_sampling
        self.snap_keep_gap = int(_settings.get().snap_keep_gap)          # QW_SNAP_KEEP_GAP: thin stored snapshots closer than this to the next one
        self.vram_snaps: List[VramSnap] = []
        self.snap_min_gap = max(BLOCK, int(_settings.get().snap_min_gap))
        self.prompt_tokens = self.reused_tokens = self.blend_candidate_tokens = 0
        self.seen_chunks = set()
        self.catch_up_rows = 0                    # MTP rows run late, after stretches without drafts
        self.last_rows: Optional[torch.Tensor] = None        # logits of the last decode / generate rows

    # ---- slots
    def num_slots(self) -> int:
        return len(self.slots)

    def slot_capacity(self, slot: int) -> int:
        return self.e.dm.slot_tokens

    def _common(self, slot: int, tokens: Sequence[int]) -> int:
        return common_prefix(self.e.slot[slot].tokens, tokens)

    def reusable(self, slot: int, tokens: Sequence[int]) -> int:
        """Tokens of the prompt the slot could keep: everything it holds when that is a prefix of the prompt."""
        c = self._common(slot, tokens)
        return c if c == len(self.e.slot[slot].tokens) and c < len(tokens) else 0

    def kept_if_chosen(self, slot: int, tokens: Sequence[int]) -> int:
        """Tokens of the prompt that need no prefill if the request goes to this slot: what the slot would continue from in
        place, or the deepest device snapshot of the slot inside what it shares with the prompt (an edited or regenerated
        last message goes back to the boundary before it).  What the block store holds is the same for every slot and
        does not enter the choice."""
        snap = self._best_vram_snapshot(slot, tokens)
        return max(self.reusable(slot, tokens), snap.n if snap is not None else 0)

    def acquire(self, tokens: Sequence[int], max_new: int) -> int:
        need = len(tokens) + max(1, max_new)
        n = len(self.slots)
        free = [not si.busy and self.slot_capacity(i) >= need for i, si in enumerate(self.slots)]
        kept = [self.kept_if_chosen(i, tokens) if free[i] else 0 for i in range(n)]
        best = H.choose_slot([si.busy for si in self.slots], [self.slot_capacity(i) for i in range(n)], kept, [si.used for si in self.slots], need)
        if best >= 0:
            self.clock += 1
            self.slots[best].busy = True
            self.slots[best].used = self.clock
        return best

    def release(self, slot: int) -> None:
        self.slots[slot].busy = False
        self.slots[slot].drafts = []

    def set_boundary_token(self, tok: int) -> None:
        self.boundary = tok

    def set_stop_tokens(self, slot: int, ids: Sequence[int]) -> None:
        self.slots[slot].stop = [int(t) for t in ids]

    # ---- prompt
    def begin_prompt(self, slot: int, tokens: Sequence[int]) -> int:
        """Make the slot ready to prefill ``tokens``: keeps what it already holds, or restores the longest stored
        prefix, or resets.  Returns the number of reused tokens."""
        si = self.slots[slot]
        toks = [int(t) for t in tokens]
        si.prompt, si.prompt_end, si.logits, si.drafts = toks, len(toks), None, []
        si.missed, si.plain_left = [], 0          # the prefill rebuilds the MTP layer's state
        for k in si.timing:
            si.timing[k] = 0.0
        self.prompt_tokens += len(toks)
        for st, ln, hs in H.chunk_prompt(toks, self.boundary):
            if hs in self.seen_chunks:
                self.blend_candidate_tokens += ln
            self.seen_chunks.add(hs)
        # four ways to start (reference: begin_keys, src/session/session.cpp:214-312): continue what the slot holds, go back to
        # a device snapshot of this slot, restore the longest stored prefix, or start from nothing - whichever keeps most
        keep = self.reusable(slot, toks)
        t0 = time.time()
        path, depth = self.store.lookup(toks[:max(0, len(toks) - 1)])      # at least one token is left to prefill
        stored = depth * BLOCK
        snap = self._best_vram_snapshot(slot, toks)
        si.last_capture = 0
        way = H.start_way(keep, snap.n if snap is not None else 0, stored)
        if way == H.START_DEVICE_SNAPSHOT:
            self._restore_vram_snapshot(slot, snap, toks)
            self.reused_tokens += snap.n
            si.last_capture = snap.n
            return snap.n
        if way == H.START_IN_PLACE:
            self.reused_tokens += keep
            self.sampler_sync(slot, toks[:keep], keep)
            si.last_capture = keep
            return keep
        self._drop_vram_snapshots(slot)
        self.e.reset(slot)
        si.block_keys = []
        self.sampler.reset_slot(slot)
        if depth == 0:
            return 0
        ok = True
        if self.pool is not None:
            # blocks travel through pinned units, eight at a time: one copy and one scatter launch per block, one wait per batch
            for b0 in range(0, depth, self.io.MAX_BATCH):
                idx = list(range(b0, min(depth, b0 + self.io.MAX_BATCH)))
                units = [self.pool.get() for _ in idx]
                try:
                    for u, bi in zip(units, idx):
                        if self.store.get_into(path[bi], u) != self.io.kv_block_bytes:
                            ok = False
                    if ok:
                        self.io.import_kv_units(slot, idx, units)
                        self.io.sync()
                finally:
                    for u in units:
                        self.pool.put(u)
                if not ok:
                    break
        else:
            for bi, key in enumerate(path[:depth]):
                kv = self.store.get(key)
                if kv is None or len(kv) != self.io.kv_block_bytes:
                    ok = False
                    break
                self.io.import_kv(slot, bi, kv)
        if ok and self.pool is not None:          # through the pinned snapshot buffer: no pageable copies
            got = self.store.get_snapshot_into(path[depth - 1], self.io._recurrent_pinned().numpy())
            if got != self.io.recurrent_bytes():
                self.e.reset(slot)
                return 0
            self.io.import_recurrent_pinned(slot)
        else:
            snap = self.store.get(path[depth - 1], snapshot=True) if ok else None
            if not ok or snap is None or len(snap[0]) != self.io.recurrent_bytes():
                self.e.reset(slot)           # a payload vanished (budget) or does not fit: recompute
                return 0
            self.io.import_recurrent(slot, snap[0])
        self.e.slot[slot].tokens = toks[:stored]
        self.e.slot[slot].mtp_hidden = None
        si.block_keys = list(path[:depth])
        self.store.note_restore(path[depth - 1], stored)
        self.reused_tokens += stored
        si.timing["restore_s"] += time.time() - t0
        self.sampler.note_tokens(slot, toks[:stored], generated=False)
        return stored

    # ---- device snapshots
    def _drop_vram_snapshots(self, slot: int) -> None:
        self.vram_snaps = [v for v in self.vram_snaps if v.slot != slot]

    def _take_vram_snapshot(self, slot: int, logits: Optional[torch.Tensor] = None) -> None:
        sl = self.e.slot[slot]
        self.vram_snaps = [v for v in self.vram_snaps if not (v.slot == slot and v.n == sl.n)]
        if len(self.vram_snaps) >= VRAM_SNAPSHOTS:
            self.vram_snaps.remove(min(self.vram_snaps, key=lambda v: v.used))
        self.clock += 1
        self.vram_snaps.append(VramSnap(slot, sl.n, self.io.snapshot_save(slot), None if sl.mtp_hidden is None else sl.mtp_hidden.clone(),
                                        None if logits is None else logits.clone(), self.clock))

    def _best_vram_snapshot(self, slot: int, toks: Sequence[int]) -> Optional[VramSnap]:
        """The deepest snapshot of this slot that lies inside what the slot and the prompt have in common (at least one
        prompt token must remain to be prefilled unless the snapshot carries the logits of its position)."""
        mine = [v for v in self.vram_snaps if v.slot == slot]
        if not mine:
            return None
        i = H.best_snapshot([v.n for v in mine], [v.logits is not None for v in mine], self._common(slot, toks), len(toks))
        return mine[i] if i >= 0 else None

    def _restore_vram_snapshot(self, slot: int, snap: VramSnap, toks: Sequence[int]) -> None:
        si, sl = self.slots[slot], self.e.slot[slot]
        self.io.snapshot_restore(slot, snap.tensors)
        sl.tokens = list(toks[:snap.n])
        sl.mtp_hidden = None if snap.mtp_hidden is None else snap.mtp_hidden.clone()
        si.block_keys = si.block_keys[:snap.n // BLOCK]
        self.clock += 1
        snap.used = self.clock
        # snapshots of later positions describe a continuation that is being abandoned
        self.vram_snaps = [v for v in self.vram_snaps if not (v.slot == slot and v.n > snap.n)]
        self.sampler_sync(slot, toks[:snap.n], snap.n)
        if snap.n == len(toks) and snap.logits is not None:
            si.logits = snap.logits.clone()

    def _capture_point(self, prompt: Sequence[int], done: int, end: int, last_capture: int) -> int:
        """Where a piece [done, end) should end so that a device snapshot can be taken at a message boundary: the last
        boundary token in the piece that lies at least ``snap_min_gap`` tokens after the previous capture (reference:
        plan_captures, src/session/prefix_cache.cpp:41-78).  ``end`` when there is none."""
        if self.boundary < 0:
            return end
        top = min(end, len(prompt) - 1)
        return H.capture_point(prompt[done:top + 1], done, len(prompt), done, end, last_capture, self.boundary, self.snap_min_gap)

    def prefetch(self, tokens: Sequence[int]) -> int:
        """Start reading, in the background, the stored blocks on the prompt's path that are only on disk, so that
        ``begin_prompt`` finds them in memory (reference: Session::prefetch, src/session/prefix_cache.cpp:34-39 and the
        load workers of src/session/block_store.cpp:312-339).  Returns the number of reads queued."""
        toks = [int(t) for t in tokens]
        path, depth = self.store.lookup(toks[:max(0, len(toks) - 1)])
        return self.store.prefetch(path[:depth], last_snapshot=True) if depth else 0

    def loads_pending(self) -> int:
        return self.store.loads_pending()

    def sampler_sync(self, slot: int, tokens: Sequence[int], prompt_end: int) -> None:
        self.sampler.reset_slot(slot)
        self.sampler.note_tokens(slot, tokens[:prompt_end], generated=False)
        self.sampler.note_tokens(slot, tokens[prompt_end:], generated=True)

    def prefill_some(self, slot: int, max_tokens: int) -> bool:
        """Prefill up to ``max_tokens`` more of the slot's prompt; True once the whole prompt is in."""
        si, sl = self.slots[slot], self.e.slot[slot]
        done = sl.n
        left = len(si.prompt) - done
        if left <= 0:
            return True
        t0 = time.time()
        n = min(left, max(1, max_tokens))
        end = done + n
        if end < len(si.prompt) and end // BLOCK * BLOCK > done:
            end = end // BLOCK * BLOCK            # pieces end on block boundaries so a snapshot can be stored there
        cap = self._capture_point(si.prompt, done, end, si.last_capture)
        at_boundary = cap < end or (cap < len(si.prompt) and si.prompt[cap] == self.boundary and cap - si.last_capture >= self.snap_min_gap)
        end = cap
        piece = si.prompt[done:end]
        last = end >= len(si.prompt)
        self.e.prefill(slot, piece, want_logits=last)
        self.sampler.note_tokens(slot, piece, generated=False)
        if last:          # the last row's logits over the whole vocabulary (gathered from the ranks' shards)
            row = self.e.last_prefill_row
            si.logits = self.e.full_logits(row + 1)[row].clone()
        if last or at_boundary:
            # the state before the next message (or before generation) stays on the device: a request that shares the prompt up to
            # here and then differs - an edited last message, a regenerated answer - goes back to it
            self._take_vram_snapshot(slot, si.logits if last else None)
            si.last_capture = end
        si.timing["prefill_s"] += time.time() - t0
        self._save_blocks(slot, snapshot=(end % BLOCK == 0))
        return last

    def _save_blocks(self, slot: int, snapshot: bool) -> None:
        """Store the slot's new full blocks; a snapshot of the recurrent state goes with the last one when the slot
        ends exactly on its boundary."""
        si, sl = self.slots[slot], self.e.slot[slot]
        if not self.store_on:
            return
        t0 = time.time()
        full = sl.n // BLOCK
        parent = si.block_keys[-1] if si.block_keys else self.store.root
        first = len(si.block_keys)
        if self.pool is not None:
            stop = False
            for b0 in range(first, full, self.io.MAX_BATCH):
                idx = list(range(b0, min(full, b0 + self.io.MAX_BATCH)))
                tw = time.time()
                units = [self.pool.get() for _ in idx]
                si.timing["pin_wait_s"] += time.time() - tw
                try:
                    self.io.export_kv_units(slot, idx, units)
                    self.io.sync()
                    for u, bi in zip(units, idx):
                        key = self.store.save_block_from(parent, bi * BLOCK, sl.tokens[bi * BLOCK:(bi + 1) * BLOCK], u.ctypes.data,
                                                         self.io.kv_block_bytes)
                        if key == 0:
                            stop = True
                            break
                        si.block_keys.append(key)
                        parent = key
                finally:
                    for u in units:
                        self.pool.put(u)
                if stop:
                    break
        else:
            for bi in range(first, full):
                toks = sl.tokens[bi * BLOCK:(bi + 1) * BLOCK]
                key = self.store.save_block(parent, bi * BLOCK, toks, self.io.export_kv(slot, bi))
                if key == 0:
                    break
                si.block_keys.append(key)
                parent = key
        if snapshot and si.block_keys and len(si.block_keys) * BLOCK == sl.n:
            anchor = sl.n < len(si.prompt) and si.prompt[sl.n] == self.boundary
            if self.pool is not None:
                addr, nb = self.io.export_recurrent_pinned(slot)
                self.store.save_snapshot_from(si.block_keys[-1], addr, nb, anchor)
            else:
                self.store.save_snapshot(si.block_keys[-1], self.io.export_recurrent(slot), None, anchor)
            if self.snap_keep_gap > 0:
                self.store.thin(self.snap_keep_gap)
        si.timing["save_s"] += time.time() - t0

    def sample_prompt(self, slot: int, p: SamplingParams) -> Tuple[int, float]:
        si = self.slots[slot]
        assert si.logits is not None, "the prompt is not in yet"
        toks, lps = self.sampler.sample(si.logits.view(1, -1), [p], [slot], [self.e.slot[slot].n],
                                        hists=[(self.e.slot[slot].tokens, si.prompt_end)])
        self.last_rows = si.logits.view(1, -1)
        return toks[0], lps[0]

    # ---- decode
    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> None:
        self.e.decode(slots, tokens, sync=False)
        for s, t in zip(slots, tokens):
            self.sampler.note_tokens(s, [int(t)], generated=True)
        self.last_rows = self.e.full_logits(len(tokens))
        self.last_row_slots = list(slots)

    def sample_row(self, row: int, p: SamplingParams) -> Tuple[int, float]:
        s = self.last_row_slots[row]
        toks, lps = self.sampler.sample(self.last_rows[row:row + 1], [p], [s], [self.e.slot[s].n],
                                        hists=[(self.e.slot[s].tokens, self.slots[s].prompt_end)])
        return toks[0], lps[0]

    def top_logprobs(self, row: int, k: int):
        lg = self.last_rows[max(row, 0)].float().cpu().numpy()
        return H.HostSampler.top_logprobs(lg, k)

    def top_logprobs_prompt(self, slot: int, k: int):
        return H.HostSampler.top_logprobs(self.slots[slot].logits.float().cpu().numpy(), k)

    # ---- generation with speculative decoding
    def draft_count(self, slot: int, k_max: int) -> int:
        return self.planner.draft_count(slot, k_max)

    def generate(self, reqs: Sequence[StepReq], k: int, force_accept: Optional[int] = None) -> List[StepOut]:
        """One step for every request: its pending token plus up to k drafts are decoded, 1..k+1 tokens are emitted.

        All requests share one draft chain (the MTP pass over one row per request, chained on the device), ONE
        verification step (the runs of all requests as consecutive rows), one sampler call over all rows and one accept
        launch (reference: src/session/generate.cpp:119-313).  Everything that can be refused - budgets, slot capacity,
        row limits - is checked before the first launch, so a ``ValueError`` leaves every slot as it was.
        ``force_accept`` (benchmarks): accept exactly that many drafts per request whatever was sampled."""
        tr = self.gen_trace
        tr.start()
        e = self.e
        # ---- plan (no state is touched here)
        max_rows = min(e.dm.max_rows, 32)
        can_draft = [bool(e.mtp and e.slot[r.slot].mtp_hidden is not None) for r in reqs]
        room = [e.dm.slot_tokens - e.slot[r.slot].n - 1 for r in reqs]
        want = self.planner.plan([r.slot for r in reqs], [r.budget for r in reqs], room, can_draft, k, e.MAX_DRAFTS, self.spec_max_rows, max_rows,
                                 forced=force_accept is not None)
        spec = e.mtp and "gdn_save" in e.dm.buf
        try:
            return self._generate_planned(reqs, want, spec, force_accept)
        except Exception as ex:
            # from here on slots may have advanced: the caller must not repeat the step for any of these requests
            raise RuntimeError(f"{self.STATE_CHANGED}: {ex}") from ex

    STATE_CHANGED = "step failed after slot state changed"

    def _generate_planned(self, reqs, want, spec, force_accept):
        tr, e = self.gen_trace, self.e
        # ---- plain stretches: a request that does not draft leaves an MTP row behind (its hidden state and pending token
        # are what the first draft row would have consumed); when its drafting resumes the rows are caught up in batches
        if e.mtp and force_accept is None:
            for i, r in enumerate(reqs):
                si, sl = self.slots[r.slot], e.slot[r.slot]
                if want[i] == 0 and si.plain_left > 0 and sl.mtp_hidden is not None:
                    si.missed.append((sl.mtp_hidden, int(r.pending), sl.n - 1))
                    del si.missed[:-MISSED_MAX]
                    self.planner.note_plain_step(r.slot)                  # at the stretch's end the next step probes with a short draft run
                elif want[i] > 0 and si.missed:
                    self.catch_up_rows += len(si.missed)
                    e.mtp_catch_up(r.slot, si.missed)
                    si.missed = []
                    tr.count("catch_up", 1)
        # ---- drafts: one chain over the requests that draft
        drafting = [i for i, kk in enumerate(want) if kk > 0]
        drafts: List[List[int]] = [[] for _ in reqs]
        if drafting:
            got = e.draft_batch([reqs[i].slot for i in drafting], [reqs[i].pending for i in drafting], max(want))
            for i, d in zip(drafting, got):
                drafts[i] = d[:want[i]]
        tr.mark("draft")
        # ---- one verification step
        slots = [r.slot for r in reqs]
        runs = [[r.pending] + drafts[i] for i, r in enumerate(reqs)]
        if spec:
            n_rows = e.verify_batch(slots, runs)
        else:
            e.decode(slots, [r.pending for r in reqs], sync=False)
            n_rows = len(reqs)
        logits = e.full_logits(n_rows).clone()
        tr.mark("verify")
        # ---- one sampler call; the pending token joins the counts first, and a row behind drafts of a request with
        # penalties is drawn on the host from the history that includes those drafts
        params, row_slots, positions, hists, force_host = [], [], [], [], []
        for i, r in enumerate(reqs):
            si, sl = self.slots[r.slot], e.slot[r.slot]
            self.sampler.note_tokens(r.slot, [r.pending], generated=True)
            base = sl.n if spec else sl.n - 1          # a plain decode step has already appended the pending token
            hist = sl.tokens[:base] + runs[i]
            for j in range(len(runs[i])):
                params.append(r.sampling)
                row_slots.append(r.slot)
                positions.append(base + j + 1)
                hists.append((hist[:base + j + 1], si.prompt_end))
                force_host.append(j > 0 and r.sampling.has_penalties())
        toks, lps = self.sampler.sample(logits, params, row_slots, positions, hists=hists, force_host=force_host)
        tr.mark("sample")
        # ---- accept per request, one launch
        outs: List[StepOut] = []
        n_acc_all, row0, keep_rows = [], 0, []
        for i, r in enumerate(reqs):
            si = self.slots[r.slot]
            d = drafts[i]
            t = toks[row0:row0 + len(runs[i])]
            # drafts that equal the tokens sampled behind them, up to a stop token; the slot's acceptance average moves
            n_acc = self.planner.accept(r.slot, t, d, si.stop, force_accept)
            if force_accept is not None:
                emitted = (d[:n_acc - 1] + [t[n_acc - 1]])[:r.budget]
            else:
                emitted = t[:n_acc][:r.budget]
            n_acc_all.append(n_acc)
            tr.count("drafts", len(d))
            tr.count("accepted", n_acc - 1)
            if self.spec_log and d:
                print(f"spec: slot {r.slot} pos {self.e.slot[r.slot].n} drafts {len(d)} accepted {n_acc - 1} rate {si.accept:.2f}", flush=True)
            stopped = bool(emitted) and emitted[-1] in si.stop
            outs.append(StepOut(emitted, lps[row0:row0 + len(emitted)], sum(n_acc_all[:-1]), stopped))
            keep_rows.append(logits[row0:row0 + n_acc])
            row0 += len(runs[i])
        if spec:
            e.accept_batch(slots, runs, n_acc_all)
        for i, r in enumerate(reqs):
            self.sampler.note_tokens(r.slot, runs[i][1:n_acc_all[i]], generated=True)
        tr.mark("accept")
        self.last_rows = torch.cat(keep_rows) if keep_rows else None
        self.last_row_slots = [r.slot for r, o in zip(reqs, outs) for _ in o.tokens]
        tr.finish()
        return outs

    # ---- stats / persistence
    def cache_stats(self) -> dict:
        s = self.store.stats()
        s.update(prompt_tokens=self.prompt_tokens, reused_tokens=self.reused_tokens,
                 blend_candidate_tokens=self.blend_candidate_tokens)
        return s

    def slot_timing(self, slot: int) -> dict:
        return dict(self.slots[slot].timing)

    def persist(self) -> None:
        """Save what the slots hold (full blocks + a snapshot where a slot ends on a block boundary) and wait for the
        disk writes."""
        for i in range(self.num_slots()):
            if self.e.slot[i].n >= BLOCK:
                self._save_blocks(i, snapshot=True)
        self.store.flush()
