"""The engine: one rank's DeviceModel plus slot bookkeeping, prefill, batched decode and chained
(device-fed) greedy decode.  With several ranks every rank process runs the same calls in the
same order (single-program, one process per GPU); collectives go through ``parallel``.

Roles of the reference's ``class Engine`` (src/engine/engine.hpp:69-446): ``prefill``, ``decode``,
slot reset, and the per-row-count decode graphs.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Tuple,  Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.ple import PleTable
from ..models.weights import Weights, synth_globals, synth_layer
from . import device_model as DM
from .device_model import DeviceModel


@dataclass
class Slot:
    tokens: List[int] = field(default_factory=list)     # every token fed so far (vision tokens negative)
    mtp_hidden: Optional[torch.Tensor] = None            # backbone hidden of the last fed position (MTP input)

    @property
    def n(self) -> int:
        return len(self.tokens)


@dataclass
class EngineOptions:
    slots: int = 1
    slot_tokens: int = 8192
    max_rows: int = DM.MAX_ROWS
    host_pages: int = 0
    dev_pages: Optional[int] = None
    save_gdn: bool = False
    use_graphs: bool = True
    prefill_rows: int = DM.MAX_ROWS          # rows per step of the row-batched prefill
    prefill_chunk: int = 4096                # tokens per chunk of the token-major (tcgen05 GEMM) prefill; 0 = off
    prefill_min: int = 64                    # shorter pieces use the row-batched path
    mtp_track: bool = False                  # plain decode steps also keep the newest hidden state for the MTP head


class Engine:
    def __init__(self, cfg: ModelConfig, opts: EngineOptions = EngineOptions(), ranks: int = 1, rank: int = 0,
                 device: str = "cuda:0"):
        self.cfg, self.opts = cfg, opts
        self.dm = DeviceModel(cfg, ranks=ranks, rank=rank, device=device, slots=opts.slots,
                              slot_tokens=opts.slot_tokens, max_rows=opts.max_rows, host_pages=opts.host_pages,
                              dev_pages=opts.dev_pages, save_gdn=opts.save_gdn)
        self.slot = [Slot() for _ in range(opts.slots)]
        self.out_host = torch.zeros(opts.max_rows, dtype=torch.int32).pin_memory()
        self.merge_argmax = None        # set by the NCCL backend: merges the ranks' (max, argmax) after a step
        self.prefiller = None           # token-major prefill, built on first use
        self.tp_channels = None         # several ranks: the prefill channels, one per micro-batch lane (parallel.tp_channel)
        self.vision_lookup = None       # vision token ids -> embeddings [n, hidden] (set by the vision front end)
        from ..utils import settings as _settings
        from ..utils.trace import ChunkProfile, StepTrace
        st = _settings.get()
        self.step_trace = StepTrace(st.trace)          # QW_TRACE: host preparation / launch / wait per row count
        self.chunk_profile = ChunkProfile(st.profile)  # QW_PROFILE: device time per prefill chunk
        self.steps = 0

    # ---- construction
    @staticmethod
    def synthetic(cfg: ModelConfig, opts: EngineOptions = EngineOptions(), ranks: int = 1, rank: int = 0,
                  device: str = "cuda:0", seed: int = 0, exact: bool = False, ple_rows: int = 1 << 20,
                  ple_pinned: bool = True, log: Optional[Callable[[str], None]] = None) -> "Engine":
        """Random-init weights of the given architecture, generated layer by layer on the device
        (a full-size model never exists in checkpoint layout in host memory)."""
        e = Engine(cfg, opts, ranks, rank, device)
        t0 = time.time()
        e.dm.set_globals(synth_globals(cfg, seed, device=device))
        for L in range(cfg.n_layers):
            e.dm.set_layer(L, synth_layer(cfg, L, seed, device=device, exact=exact))
            if log and (L % 8 == 7 or L == cfg.n_layers - 1):
                log(f"layer {L + 1}/{cfg.n_layers} ready, {e.dm.weight_bytes() / 1e9:.1f} GB, {time.time() - t0:.0f} s")
        table = PleTable.synthetic(cfg, rows=ple_rows, layout="f8", seed=seed, pin=ple_pinned)
        e.dm.set_ple_table(table)
        if cfg.mtp:
            g = synth_globals(cfg, seed, device=device)
            g.update(synth_layer(cfg, cfg.n_layers, seed, device=device, exact=exact, prefix="mtp.layers.0.", qsa=True))
            e.dm.set_mtp(g)
        torch.cuda.synchronize(device)
        return e

    @staticmethod
    def from_weights(cfg: ModelConfig, w: Weights, table: Optional[PleTable], opts: EngineOptions = EngineOptions(),
                     ranks: int = 1, rank: int = 0, device: str = "cuda:0") -> "Engine":
        e = Engine(cfg, opts, ranks, rank, device)
        e.dm.set_globals(w)
        for L in range(cfg.n_layers):
            e.dm.set_layer(L, w)
        if table is not None:
            e.dm.set_ple_table(table)
        if cfg.mtp and "mtp.fc_hidden.weight" in w:
            e.dm.set_mtp(w)
        return e

    @staticmethod
    def from_checkpoint(cfg: ModelConfig, model_dir: str, table: Optional[PleTable], opts: EngineOptions = EngineOptions(),
                        ranks: int = 1, rank: int = 0, device: str = "cuda:0", weight_cache_dir: Optional[str] = None,
                        log=None) -> "Engine":
        """Load a checkpoint directory.  With ``weight_cache_dir`` the converted per-rank tensors are written to
        ``rank<r>.qww`` the first time and read back on later starts without touching the checkpoint
        (reference: src/engine/weights.hip:33-176)."""
        from ..models.weights import load_checkpoint
        from .weight_cache import WeightCache, cache_key
        e = Engine(cfg, opts, ranks, rank, device)
        wc = None
        if weight_cache_dir:
            shapes = repr(sorted((k, v) for k, v in cfg.__dict__.items() if isinstance(v, (int, float, bool, tuple))))
            wc = WeightCache(weight_cache_dir, rank, cache_key(model_dir, rank, ranks, shapes))
            e.dm.weight_cache = wc
            if log:
                log(f"weight cache {wc.path}: {'replaying' if wc.replaying else 'recording'}")
        w = None if (wc is not None and wc.replaying) else load_checkpoint(cfg, model_dir)
        e.dm.set_globals(w)
        for L in range(cfg.n_layers):
            e.dm.set_layer(L, w)
        has_mtp = cfg.mtp
        if has_mtp:
            present = e.dm._cached("mtp_present", lambda: {"present": bool(w is not None and "mtp.fc_hidden.weight" in w)})
            if present["present"]:
                e.dm.set_mtp(w)
        if wc is not None:
            wc.close()
            e.dm.weight_cache = None
        if table is not None:
            e.dm.set_ple_table(table)
        return e

    # ---- start-up: memory plan and graph warm-up
    def memory_plan(self) -> Dict[str, float]:
        """GB this rank holds (weights, KV + recurrent state, step buffers) and what the device has; raises when the plan
        does not fit with 2 GB to spare (the reference checks its VRAM plan before loading: src/engine/engine.hip:125-163)."""
        dm = self.dm
        gb = lambda ts: sum(t.numel() * t.element_size() for t in ts) / 2**30
        state = gb(dm.k_dev + dm.v_dev + dm.ck + dm.raw_ring + dm.gdn_S + dm.gdn_ring + [dm.ple_ring])
        plan = {"weights_gb": dm.weight_bytes() / 2**30, "state_gb": state, "buffers_gb": gb(list(dm.buf.values())),
                "host_kv_gb": gb((dm.k_host or []) + (dm.v_host or []))}
        free, total = torch.cuda.mem_get_info(dm.dev)
        plan["device_total_gb"], plan["device_free_gb"] = total / 2**30, free / 2**30
        if free < 2 * 2**30:
            raise RuntimeError(f"memory plan leaves {free / 2**30:.1f} GB free on {dm.dev}: {plan}")
        return plan

    def warmup(self, max_rows: int = 8, spec: bool = True) -> int:
        """Capture every graph a request can need before the first request arrives: plain steps of 1..max_rows rows, the
        verification form of the same (GDN state saves, hidden states kept) and the chained MTP pass; returns the number of
        graphs held.  Runs on slot 0, which is reset afterwards (reference: src/engine/engine.hip:276-312 captures every
        graph at start for the same reason: a capture in front of a user costs tens of milliseconds)."""
        if not self.opts.use_graphs:
            return 0
        self.reset(0)
        kinds = [0]
        if spec and self.opts.save_gdn:
            kinds.append(DM.FLAG_SAVE_GDN | DM.FLAG_KEEP_HIDDEN)
        for flags in kinds:
            for m in range(1, max_rows + 1):
                base = self.slot[0].n
                toks = [5 + i for i in range(m)]
                for _ in range(2):          # first call captures (and runs once), second call replays
                    self.dm.step(toks, [0] * m, list(range(base, base + m)), self._ctx3(0, toks), flags=flags, graph=True)
        if self.merge_argmax is None:
            self.decode_chain(0, 5, 2)
        if spec and self.mtp and self.opts.save_gdn:
            self.reset(0)
            self.prefill(0, [5, 6, 7, 8])
            self.generate_greedy(0, 9, 4, k=2)
        torch.cuda.synchronize(self.dm.dev)
        self.dm.check_error()
        self.reset(0)
        return len(self.dm.graphs)

    # ---- slots
    def reset(self, slot: int):
        self.slot[slot] = Slot()
        self.dm.reset_slot(slot)

    def _ctx3(self, slot: int, toks: Sequence[int]) -> np.ndarray:
        c = self.cfg
        hist = [c.real_token(t) for t in self.slot[slot].tokens[-2:]]
        seq = hist + [c.real_token(int(t)) for t in toks]
        out = np.full((len(toks), 3), -1, dtype=np.int32)
        for i in range(len(toks)):
            p = len(hist) + i
            out[i, 0] = seq[p]
            if p >= 1:
                out[i, 1] = seq[p - 1]
            if p >= 2:
                out[i, 2] = seq[p - 2]
        return out

    # ---- prefill (row-batched: the decode kernels over runs of up to prefill_rows rows)
    def prefill(self, slot: int, tokens: Sequence[int], want_logits: bool = True) -> Optional[torch.Tensor]:
        """Append ``tokens`` to the slot.  Returns the logits of the last token (device tensor)."""
        toks = [int(t) for t in tokens]
        n = len(toks)
        has_media = any(t < 0 for t in toks)
        token_major = self.opts.prefill_chunk > 0 and (self.dm.sc.ranks == 1 or self.tp_channels is not None)
        if has_media and (self.vision_lookup is None or not token_major):
            raise ValueError("vision tokens need a vision tower and the token-major prefill path")
        if token_major and (n >= self.opts.prefill_min or has_media):
            return self._prefill_token_major(slot, toks, want_logits)
        step = max(1, min(self.opts.prefill_rows, self.opts.max_rows))
        i = 0
        while i < n:
            chunk = toks[i:i + step]
            base = self.slot[slot].n
            if base + len(chunk) > self.dm.slot_tokens:
                raise ValueError("slot capacity exceeded")
            last = i + len(chunk) >= n
            flags = 0 if (last and want_logits) else DM.FLAG_NO_HEAD
            if self.mtp:
                flags |= DM.FLAG_KEEP_HIDDEN
            self.dm.step(chunk, [slot] * len(chunk), list(range(base, base + len(chunk))), self._ctx3(slot, chunk),
                         flags=flags, graph=False)
            if self.mtp:
                self._mtp_rows(slot, base, chunk)
            self.slot[slot].tokens.extend(chunk)
            i += len(chunk)
        self.steps += 1
        if want_logits:
            if self.merge_argmax is not None:
                self.merge_argmax(len(chunk))
            self.last_prefill_row = (n - 1) % step if n % step else step - 1
            return self.dm.buf["logits"][self.last_prefill_row]
        return None

    # ---- MTP / speculative decoding (one GPU)
    @property
    def mtp(self) -> bool:
        return bool(self.dm.model.mtp.enabled)

    def _mtp_rows(self, slot: int, base: int, chunk: List[int]):
        """After a backbone step over ``chunk`` at positions base.. (hidden states in buf['hidden_out']): run the MTP
        rows whose next token is known (all but the last), first the row left over from the previous call."""
        dm, sl = self.dm, self.slot[slot]
        hid = dm.buf["hidden_out"]
        n = len(chunk)
        keep = hid[n - 1].clone()
        # logits / argmax of the backbone step must survive the MTP pass
        saved = (dm.buf["logits"][:n].clone(), dm.buf["amax_idx"][:n].clone(), dm.buf["amax_val"][:n].clone())
        if sl.mtp_hidden is not None and base > 0:
            # shift the rows down by one and put the pending hidden in front: rows = positions base-1 .. base+n-2
            hid[1:n] = hid[0:n - 1].clone()
            hid[0] = sl.mtp_hidden
            dm.mtp_step(chunk, [slot] * n, list(range(base - 1, base - 1 + n)))
        elif n > 1:
            dm.mtp_step(chunk[1:], [slot] * (n - 1), list(range(base, base + n - 1)))
        sl.mtp_hidden = keep
        dm.buf["logits"][:n].copy_(saved[0])
        dm.buf["amax_idx"][:n].copy_(saved[1])
        dm.buf["amax_val"][:n].copy_(saved[2])

    def draft(self, slot: int, pending: int, k: int) -> List[int]:
        """k greedy draft tokens after ``pending`` (the sampled token that has not been decoded yet): one MTP row
        from the backbone hidden of the last position, then chained rows from the MTP's own hidden."""
        dm, sl = self.dm, self.slot[slot]
        assert self.mtp and sl.mtp_hidden is not None
        dm.buf["hidden_out"][0] = sl.mtp_hidden
        pos = sl.n - 1
        if self.opts.use_graphs and k > 1:
            # chained: the graph of one MTP pass ends by feeding its token, position and hidden state to the next pass
            # on the device, so k drafts are k graph replays and one read-back
            flags = DM.FLAG_CHAIN
            key = ("mtp", 1, flags)
            got = torch.zeros(k, dtype=torch.int32, device=dm.dev)
            if key not in dm.graphs:
                dm.mtp_step([pending], [slot], [pos], flags=flags, graph=True)       # captures; the warm-up is the first pass
                got[0:1].copy_(dm.buf["amax_idx"][0:1])
                done = 1
            else:
                dm.stage_rows([pending], [slot], [pos], None)
                done = 0
            g = dm.graphs[key]
            for j in range(done, k):
                g.replay()
                got[j:j + 1].copy_(dm.buf["amax_idx"][0:1], non_blocking=True)
            torch.cuda.current_stream(dm.dev).synchronize()
            return got.tolist()
        out, tok = [], pending
        for j in range(k):
            dm.mtp_step([tok], [slot], [pos + j], graph=self.opts.use_graphs)
            tok = int(dm.buf["amax_idx"][0])
            out.append(tok)
        return out

    def verify(self, slot: int, rows: List[int]) -> torch.Tensor:
        """Decode ``rows`` = [pending, draft 1, ...] as one run, keeping the GDN state after every row and the hidden
        states.  Returns the logits [len(rows), vocab] (device)."""
        dm = self.dm
        base = self.slot[slot].n
        n = len(rows)
        dm.step(rows, [slot] * n, list(range(base, base + n)), self._ctx3(slot, rows),
                flags=DM.FLAG_SAVE_GDN | DM.FLAG_KEEP_HIDDEN, graph=self.opts.use_graphs)
        return dm.buf["logits"][:n]

    def accept(self, slot: int, rows: List[int], n_acc: int):
        """Keep the first ``n_acc`` rows of the last verify: the GDN state after row n_acc-1 becomes the slot's state."""
        dm, sl = self.dm, self.slot[slot]
        if n_acc < len(rows):
            save = dm.buf["gdn_save"]
            for gi in range(self.cfg.n_gdn):
                dm.gdn_S[gi][slot].copy_(save[gi, n_acc - 1])
        base = sl.n
        sl.mtp_hidden = dm.buf["hidden_out"][n_acc - 1].clone()
        if n_acc == len(rows) and n_acc >= 2:
            # every draft was accepted: the MTP layer has no row yet for the position of the last-but-one row
            # (its next token, the last draft, is only now confirmed)
            dm.buf["hidden_out"][0] = dm.buf["hidden_out"][n_acc - 2].clone()
            dm.mtp_step([rows[n_acc - 1]], [slot], [base + n_acc - 2])
        sl.tokens.extend(int(t) for t in rows[:n_acc])

    # ---- the same for several requests at once (one draft chain, one verification step, one accept launch)
    MAX_DRAFTS = min(DM.GDN_RING, DM.RAW_RING) - 4      # a verification run longer than this would wrap the rings a rollback needs

    def full_logits(self, n: int) -> torch.Tensor:
        """Rows 0..n-1 of the last step's logits over the whole vocabulary [n, vocab] (device).  With several ranks the
        vocabulary shards are gathered into every rank's copy first (one collective outside the step's graph)."""
        dm = self.dm
        if dm.sc.ranks == 1 or getattr(dm, "logits_full", None) is None:
            return dm.buf["logits"][:n]
        s = torch.cuda.current_stream(dm.dev).cuda_stream
        import ctypes as C
        rc = dm.lib.qwrt_gather_logits(C.byref(dm.model), n, 4000, C.c_void_p(s))
        if rc != 0:
            raise RuntimeError(f"qwrt_gather_logits failed: {rc}")
        return dm.logits_full[:n]

    def draft_batch(self, slots: Sequence[int], pendings: Sequence[int], k: int) -> List[List[int]]:
        """k greedy draft tokens for every request (row i: slot ``slots[i]``, not yet decoded token ``pendings[i]``): one
        MTP pass over all requests, chained k times on the device, one read-back."""
        dm = self.dm
        M = len(slots)
        if M == 0 or k <= 0:
            return [[] for _ in slots]
        k = min(k, self.MAX_DRAFTS)
        hid = dm.buf["hidden_out"]
        for i, s_ in enumerate(slots):
            assert self.slot[s_].mtp_hidden is not None
            hid[i].copy_(self.slot[s_].mtp_hidden)
        pos = [self.slot[s_].n - 1 for s_ in slots]
        got = torch.zeros((k, M), dtype=torch.int32, device=dm.dev)
        if self.opts.use_graphs:
            flags = DM.FLAG_CHAIN
            key = ("mtp", M, flags)
            if key not in dm.graphs:
                dm.mtp_step(list(pendings), list(slots), pos, flags=flags, graph=True)       # captures; the warm-up is the first pass
                got[0].copy_(dm.buf["amax_idx"][:M])
                done = 1
            else:
                dm.stage_rows(list(pendings), list(slots), pos, None)
                done = 0
            g = dm.graphs[key]
            for j in range(done, k):
                g.replay()
                got[j].copy_(dm.buf["amax_idx"][:M], non_blocking=True)
        else:
            toks = list(pendings)
            for j in range(k):
                dm.mtp_step(toks, list(slots), [p + j for p in pos])
                got[j].copy_(dm.buf["amax_idx"][:M])
                toks = got[j].tolist()
        torch.cuda.current_stream(dm.dev).synchronize()
        cols = got.t().tolist()
        return [list(c) for c in cols]

    def verify_batch(self, slots: Sequence[int], runs: Sequence[List[int]]) -> int:
        """One step over the runs of all requests (``runs[i]`` = [pending, draft 1, ...] appended to ``slots[i]``), keeping
        the GDN state after every row and the hidden states.  Returns the number of rows; logits / argmax are in the
        step buffers, the rows of a request consecutive and in request order."""
        row_slots, row_toks, row_pos = [], [], []
        c3 = []
        for s_, run in zip(slots, runs):
            base = self.slot[s_].n
            if base + len(run) > self.dm.slot_tokens:
                raise ValueError("slot capacity exceeded")
            row_slots += [s_] * len(run)
            row_toks += [int(t) for t in run]
            row_pos += list(range(base, base + len(run)))
            c3.append(self._ctx3(s_, run))
        n = len(row_toks)
        if n > self.dm.max_rows:
            raise ValueError("too many rows in one verification step")
        self.dm.step(row_toks, row_slots, row_pos, np.concatenate(c3), flags=DM.FLAG_SAVE_GDN | DM.FLAG_KEEP_HIDDEN,
                     graph=self.opts.use_graphs)
        return n

    def accept_batch(self, slots: Sequence[int], runs: Sequence[List[int]], n_acc: Sequence[int]) -> None:
        """Keep the first ``n_acc[i]`` rows of request i of the last ``verify_batch``: one launch copies the saved GDN states
        of all requests and layers; requests whose drafts were all accepted get the MTP row they still lack."""
        import ctypes as C
        dm = self.dm
        if not hasattr(self, "_accept_pairs"):
            self._accept_pairs_host = torch.zeros(2 * dm.max_rows, dtype=torch.int32).pin_memory()
            self._accept_pairs = torch.zeros(2 * dm.max_rows, dtype=torch.int32, device=dm.dev)
            self._gdn_ptrs = torch.tensor([t.data_ptr() for t in dm.gdn_S] or [0], dtype=torch.int64, device=dm.dev)
        h = self._accept_pairs_host.numpy()
        row0, catch = 0, []
        hid = dm.buf["hidden_out"]
        for i, (s_, run, na) in enumerate(zip(slots, runs, n_acc)):
            h[2 * i], h[2 * i + 1] = s_, (row0 + na - 1) if na < len(run) else -1
            sl = self.slot[s_]
            sl.mtp_hidden = hid[row0 + na - 1].clone()
            if na == len(run) and na >= 2:
                catch.append((s_, row0 + na - 2, run[na - 1], sl.n + na - 2))
            row0 += len(run)
        if self.cfg.n_gdn and "gdn_save" in dm.buf and any(h[2 * i + 1] >= 0 for i in range(len(slots))):
            self._accept_pairs.copy_(self._accept_pairs_host, non_blocking=True)
            st = C.c_void_p(torch.cuda.current_stream(dm.dev).cuda_stream)
            state = dm.sc.gdn_vl * self.cfg.gdn_dim * self.cfg.gdn_dim
            rc = dm.lib.qwk_gdn_accept(C.c_void_p(self._gdn_ptrs.data_ptr()), C.c_void_p(dm.buf["gdn_save"].data_ptr()), self.cfg.n_gdn,
                                       dm.max_rows, state, C.c_void_p(self._accept_pairs.data_ptr()), len(slots), st)
            if rc != 0:
                raise RuntimeError(f"qwk_gdn_accept failed: {rc}")
        if catch and self.mtp:
            # every draft was accepted: the MTP layer has no row yet for the position of the last-but-one row
            rows_h = torch.stack([hid[r].clone() for _, r, _, _ in catch])
            hid[:len(catch)].copy_(rows_h)
            dm.mtp_step([t for _, _, t, _ in catch], [s_ for s_, _, _, _ in catch], [p for _, _, _, p in catch])
        for s_, run, na in zip(slots, runs, n_acc):
            self.slot[s_].tokens.extend(int(t) for t in run[:na])

    def mtp_catch_up(self, slot: int, rows: Sequence[Tuple[torch.Tensor, int, int]]) -> int:
        """MTP rows that were skipped while the slot decoded without drafts: ``rows`` = (backbone hidden state of position
        p, token of position p + 1, p) in position order.  They run as batched MTP passes (up to ``max_rows`` rows each), so
        that the MTP layer's own KV / indexer state has no holes when drafting resumes.  Returns the number of passes.
        (reference: mtp_catch_up, src/engine/speculative.hip:43-66)"""
        if not self.mtp or not rows:
            return 0
        dm, hid = self.dm, self.dm.buf["hidden_out"]
        step, passes = dm.max_rows, 0
        for i in range(0, len(rows), step):
            part = rows[i:i + step]
            hid[:len(part)].copy_(torch.stack([h for h, _, _ in part]))
            dm.mtp_step([int(t) for _, t, _ in part], [slot] * len(part), [int(p_) for _, _, p_ in part])
            passes += 1
        return passes

    def generate_greedy(self, slot: int, pending: int, n_new: int, k: int = 0) -> List[int]:
        """Greedy continuation of ``n_new`` tokens; with k > 0 drafts are verified (the result equals k = 0)."""
        out: List[int] = []
        self.spec_steps = self.spec_accepted = 0
        while len(out) < n_new:
            if k <= 0 or not self.mtp:
                pending = self.decode([slot], [pending])[0]
                out.append(pending)
                continue
            drafts = self.draft(slot, pending, k)
            rows = [pending] + drafts
            self.verify(slot, rows)
            picks = self.dm.buf["amax_idx"][:len(rows)].tolist()          # merged over the vocabulary shards on the device
            n_acc = 1
            while n_acc <= k and picks[n_acc - 1] == drafts[n_acc - 1]:
                n_acc += 1
            self.accept(slot, rows, n_acc)
            out.extend(picks[:n_acc])
            pending = picks[n_acc - 1]
            self.spec_steps += 1
            self.spec_accepted += n_acc - 1
        return out[:n_new]

    def _get_prefiller(self):
        from .prefill import Prefiller
        if self.prefiller is None:
            self.prefiller = Prefiller(self.dm, chunk=min(self.opts.prefill_chunk, max(256, self.dm.slot_tokens)),
                                       channels=self.tp_channels)
        return self.prefiller

    def prefill_jobs(self, slot: int, toks: List[int], want_logits: bool):
        """The token-major prefill of ``toks`` as a generator: yields the job of each chunk (``QwPrefillJob``), which the
        caller launches before resuming.  One process per GPU launches each job by itself (``_prefill_token_major``); a
        process that emulates several ranks on one GPU launches the ranks' jobs of a chunk together."""
        if self.slot[slot].n + len(toks) > self.dm.slot_tokens:
            raise ValueError("slot capacity exceeded")
        pf = self._get_prefiller()
        T = pf.T
        for i in range(0, len(toks), T):
            chunk = toks[i:i + T]
            last = i + T >= len(toks)
            sl = self.slot[slot]
            base = sl.n
            embeds = None
            vis = [j for j, t in enumerate(chunk) if t < 0]
            if vis:         # rows that carry vision tokens take the tower's output as their embedding
                embeds = (torch.tensor(vis, dtype=torch.long, device=self.dm.dev), self.vision_lookup([chunk[j] for j in vis]))
            ev = self.chunk_profile.begin()
            if pf.native:
                yield pf.make_job(slot, base, chunk, self._ctx3(slot, chunk), want_logits and last, embeds, mtp=self.mtp,
                                  pending=sl.mtp_hidden)
                if self.mtp:
                    sl.mtp_hidden = pf.b["hid_out"].clone()
            else:
                pf.run_py(slot, base, chunk, self._ctx3(slot, chunk), want_logits and last, embeds=embeds)
                if self.mtp:
                    # the chunk's hidden states are in the prefiller's X: MTP rows for every position whose next token is known
                    keep = pf.b["X"][len(chunk) - 1].clone()
                    if want_logits and last:             # the MTP rows below reuse the logits / argmax buffers
                        saved = (self.dm.buf["logits"][:1].clone(), self.dm.buf["amax_idx"][:1].clone())
                    if sl.mtp_hidden is not None and base > 0:
                        self.dm.buf["hidden_out"][0] = sl.mtp_hidden
                        self.dm.mtp_step([chunk[0]], [slot], [base - 1])
                    pf.mtp_pass(slot, base, len(chunk), chunk[1:])
                    if want_logits and last:
                        self.dm.buf["logits"][:1].copy_(saved[0])
                        self.dm.buf["amax_idx"][:1].copy_(saved[1])
                    sl.mtp_hidden = keep
            self.chunk_profile.end(ev, len(chunk))
            sl.tokens.extend(chunk)
        self.steps += 1
        self.chunk_profile.summary(f"prefill slot {slot}")
        self.last_prefill_row = 0           # logits / argmax of the last token sit in row 0

    def _prefill_token_major(self, slot: int, toks: List[int], want_logits: bool):
        from .prefill import Prefiller
        for job in self.prefill_jobs(slot, toks, want_logits):
            self._rendezvous()
            Prefiller.launch(self.dm.lib, [job])
        return self.dm.buf["logits"][0] if want_logits else None

    def _rendezvous(self) -> None:
        """Several ranks, one process each: a one-element all-reduce on the stream before a chunk's kernels.  The kernels'
        own waits for their peers are bounded (about a second), which covers the ranks' differences in kernel time but not
        a rank whose host is late by more - a first call that still allocates buffers or loads kernels, a worker process
        that got its call over a socket; behind the all-reduce both GPUs start the chunk together wherever their hosts are."""
        if self.dm.sc.ranks == 1:
            return
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() != self.dm.sc.ranks:
            return          # ranks emulated in one process are walked in lock step by the runtime
        if getattr(self, "_rdv", None) is None:
            self._rdv = torch.zeros(1, device=self.dm.dev)
        dist.all_reduce(self._rdv)

    # ---- decode
    def decode(self, slots: Sequence[int], tokens: Sequence[int], flags: int = 0, sync: bool = True) -> List[int]:
        """One batched step: row i appends tokens[i] to slots[i] (rows of a slot consecutive).
        Returns the greedy next token of every row (host ints)."""
        M = len(tokens)
        self.step_trace.begin()
        pos, c3 = [], []
        seen: Dict[int, int] = {}
        for s, t in zip(slots, tokens):
            k = seen.get(s, 0)
            pos.append(self.slot[s].n + k)
            seen[s] = k + 1
        # n-gram context per row, following the run inside the batch
        tmp = {s: list(self.slot[s].tokens[-2:]) for s in seen}
        rows3 = np.full((M, 3), -1, dtype=np.int32)
        for i, (s, t) in enumerate(zip(slots, tokens)):
            h = tmp[s]
            rows3[i, 0] = self.cfg.real_token(int(t))
            if len(h) >= 1:
                rows3[i, 1] = self.cfg.real_token(h[-1])
            if len(h) >= 2:
                rows3[i, 2] = self.cfg.real_token(h[-2])
            h.append(int(t))
        track = self.mtp and self.opts.mtp_track
        if track:
            flags |= DM.FLAG_KEEP_HIDDEN
        self.step_trace.launched()
        self.dm.step(list(tokens), list(slots), pos, rows3, flags=flags, graph=self.opts.use_graphs)
        self.step_trace.enqueued()
        if track:
            # plain steps leave the MTP layer one row behind per token: remember the newest hidden per slot; the rows in
            # between are caught up by _mtp_rows the next time drafts are wanted (here: simply dropped for rows > 1 back)
            for i, s_ in enumerate(slots):
                self.slot[s_].mtp_hidden = self.dm.buf["hidden_out"][i].clone()
        for s, t in zip(slots, tokens):
            self.slot[s].tokens.append(int(t))
        self.steps += 1
        if self.merge_argmax is not None:
            self.merge_argmax(M)            # vocabulary-parallel argmax merged outside the graph (NCCL backend)
        self.out_host[:M].copy_(self.dm.buf["amax_idx"][:M], non_blocking=True)
        if sync:
            torch.cuda.current_stream(self.dm.dev).synchronize()
            self.step_trace.end(M)
            return self.out_host[:M].tolist()
        return []

    def decode_chain(self, slot: int, first_token: int, n_steps: int) -> List[int]:
        """Greedy-decode ``n_steps`` tokens of one slot with the token fed back on the device: the
        graph of one step (with the row-advance kernel at its end) is replayed ``n_steps`` times with
        no host work in between; the sampled tokens are read back once at the end."""
        dm = self.dm
        if self.merge_argmax is not None:
            raise RuntimeError("chained decode needs the device-side argmax merge (p2p backend)")
        base = self.slot[slot].n
        if base + n_steps > dm.slot_tokens:
            raise ValueError("slot capacity exceeded")
        flags = DM.FLAG_CHAIN
        key = (1, flags, -1)
        out = torch.zeros(n_steps, dtype=torch.int32, device=dm.dev)
        if key not in dm.graphs:
            # capture on this slot's real state: the warm-up launch is the first step
            dm.step([first_token], [slot], [base], self._ctx3(slot, [first_token]), flags=flags, graph=True)
            out[0:1].copy_(dm.buf["amax_idx"][0:1])
            done = 1
        else:
            dm.stage_rows([first_token], [slot], [base], self._ctx3(slot, [first_token]))
            done = 0
        g = dm.graphs[key]
        for i in range(done, n_steps):
            g.replay()
            out[i:i + 1].copy_(dm.buf["amax_idx"][0:1], non_blocking=True)
        torch.cuda.current_stream(dm.dev).synchronize()
        toks = out.tolist()
        self.slot[slot].tokens.extend([first_token] + toks[:-1])
        self.steps += n_steps
        return toks
