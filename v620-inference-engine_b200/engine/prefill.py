"""Token-major prefill of one slot: a chunk of T prompt tokens through the whole model.

Every dense product runs on the tcgen05 GEMM (``qwk_gemm_bf16_tc``), the routed experts as one grouped tcgen05
GEMM per projection over expert-sorted rows with the q4 words converted inside the kernel, and the stateful
pieces (GDN conv + chunked scan, QSA prep / indexer / selection / attention over the paged KV, PLE) on kernels
that leave the slot state exactly as the decode kernels expect it (reference: ``run_prefill_rank``,
src/engine/prefill.hip:46-496).

The chunk's launch sequence lives in the native runtime (``ops/csrc/prefill_rt.cu``, one call per chunk): one rank
or several (tensor + expert parallel with the collectives inside the kernels, ``ops/csrc/tp.cuh``), one or two
micro-batches on two streams.  This module owns the buffers (PyTorch allocations), the row tables and the job
struct.  ``run_py`` keeps the same schedule spelled out in Python, kernel by kernel, for one GPU: the cross-check
of the runtime in the tests, and ``QW_PREFILL_PY=1``.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import lib as qlib
from ..ops import structs as S
from ..utils import settings
from . import device_model as DM
from .device_model import DeviceModel

P = C.c_void_p


def _p(t):
    return None if t is None else P(t.data_ptr())


class Prefiller:
    def __init__(self, dm: DeviceModel, chunk: int = 4096, attn_rows: int = 256, channels=None, lanes: int = 0):
        """``channels``: with several ranks, one ``TpChannel`` per micro-batch lane (``parallel/tp_channel.py``)."""
        st = settings.get()
        self.dm, self.T, self.attn_rows = dm, chunk, attn_rows
        self.on_block_input = None      # optional hook(layer, "attn" | "mlp", block input [n, hidden] bf16): calibration
        self.layer_limit = None         # run only the first n layers, then the final mixer (depth diagnostics)
        self.lib = dm.lib
        self.channels = list(channels or [])
        self.tp = dm.sc.ranks > 1
        if self.tp and not self.channels:
            raise ValueError("token-major prefill on several ranks needs a channel per lane (parallel.tp_channel)")
        self.lanes = lanes or st.prefill_lanes or (len(self.channels) if self.tp else 1)          # attach_tp made one channel per lane
        self.lanes = max(1, min(self.lanes, len(self.channels))) if self.tp else self.lanes
        S.check_prefill_structs(self.lib)
        self.lib.qwrt_prefill.argtypes = [C.POINTER(C.POINTER(S.QwPrefillJob)), C.c_int]
        self.lib.qwrt_prefill.restype = C.c_int
        self.lib.qwrt_prefill_last_launches.restype = C.c_longlong
        c, sc, dev = dm.cfg, dm.sc, dm.dev
        T = chunk
        f32, bf, i32 = torch.float32, torch.bfloat16, torch.int32
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        self.hc_ld = (c.hc_down + 7) // 8 * 8
        K_down = c.hc * sc.sh
        kblocks = (K_down + 63) // 64
        self.hc_ksplit = 3 if (kblocks >= 48 and not self.tp) else 1          # split-K shares of the mixers' down projection
        if (kblocks + self.hc_ksplit - 1) // self.hc_ksplit * (self.hc_ksplit - 1) >= kblocks:
            self.hc_ksplit = 1
        nrs = c.n_experts + 1 + 2 * sc.sffn_l
        self.nrs_ld = (nrs + 7) // 8 * 8
        self.proj_ld = (max(sc.gdn_proj_l, sc.qsa_proj_l) + 7) // 8 * 8
        self.o_ld = max(sc.gdn_vl * c.gdn_dim, sc.qh_l * c.head_dim)
        self.ple_ld = (sc.ple_kv + 7) // 8 * 8
        Pn = T * c.top_k
        self.max_tiles = Pn // 128 + sc.exp_l
        nch = (T + 63) // 64 + 1
        self.gdn_scratch_lane = nch * sc.gdn_vl * (2 * 64 * 128 + 64 * 64 + 64) + T * sc.gdn_vl * 128
        one = not self.tp
        self.b = {
            "X": z((T, c.hc, sc.sh), f32), "xn": z((T, c.hc * sc.sh), bf), "d": z((self.hc_ksplit, T, self.hc_ld), f32) if one else None,
            "u": z((T, c.hc_rank), bf), "inj_a": z((T, c.hc), f32), "inj_b": z((T, c.hc), f32), "g": z((T, c.hc * sc.sh), f32),
            "bin": z((T, c.hidden), bf) if one else None,
            "proj": z((T, self.proj_ld), f32), "o": z((T, self.o_ld), bf),
            "out_a": z((T, c.hidden), f32) if one else None, "out_b": z((T, c.hidden if one else sc.sh), f32),
            "qkv": z((T, sc.gdn_qkv_l), f32), "decay": z((T, sc.gdn_vl), f32), "beta": z((T, sc.gdn_vl), f32),
            "q": z((T, sc.qh_l, c.head_dim), f32), "iq": z((T, c.idx_heads, c.idx_dim), f32),
            "scores": z((T, dm.model.d.score_cap), f32), "sel": z((T, c.idx_topk_blocks), i32), "sel_n": z((T,), i32),
            "rs": z((T, self.nrs_ld), f32), "pe": z((T, c.top_k), i32), "pw": z((T, c.top_k), f32),
            "sh_h": z((T, sc.sffn_l), bf), "sd": z((T, c.hidden), f32),
            "xperm": z((Pn + 128, c.hidden), bf), "h13": z((Pn, 2 * c.ffn), bf), "h": z((Pn + 128, c.ffn), bf),
            "y": z((Pn, c.hidden), f32),
            "ple_e": z((T, c.hidden), bf), "ple_kv": z((T, self.ple_ld), f32), "ple_send": z((T, 16), f32), "ple_red": z((T, 16), f32),
            "ple_gv": z((T, sc.xw), f32), "ple_nc": z((T, sc.xw), f32),
            "rows": z((11 * T,), i32),
            "inv": z((Pn,), i32), "src_token": z((Pn,), i32),
            "t13": z((2 * self.max_tiles, 4), i32), "t2": z((2 * self.max_tiles, 4), i32),
            "gdn_scratch": z((2 * self.gdn_scratch_lane,), f32),
            "hid_out": z((c.hc, sc.sh), f32), "amax16": z((16,), f32),
        }
        # the run_py path keeps the decode kernels' attention scratch
        self.gdn_chunked = not st.gdn_sequential
        self.qsa_mma = not st.qsa_attend_rows and sc.qh_l // sc.kvh_l <= 16
        self.q4_fused = not st.moe_dequant_scratch and c.hidden % 128 == 0 and c.ffn % 128 == 0
        # the native runtime covers the default forms of the kernels; the diagnostic forms run from Python
        self.native = (not st.prefill_py and self.gdn_chunked and self.qsa_mma and self.q4_fused) or self.tp
        if self.tp and not (self.gdn_chunked and self.qsa_mma and self.q4_fused):
            raise ValueError("QW_GDN_SEQUENTIAL / QW_QSA_ATTEND_ROWS / QW_MOE_DEQUANT_SCRATCH are one-GPU diagnostics")
        if not self.native:
            if not self.qsa_mma:
                nsp = dm.model.d.nsplit
                self.b["pm"], self.b["pl"] = z((attn_rows, sc.qh_l, nsp), f32), z((attn_rows, sc.qh_l, nsp), f32)
                self.b["pacc"] = z((attn_rows, sc.qh_l, nsp, c.head_dim), f32)
            if not self.q4_fused:
                self.b["w13dq"] = z((sc.exp_l * 2 * c.ffn, c.hidden), bf)
                self.b["w2dq"] = z((sc.exp_l * c.hidden, c.ffn), bf)
        # ring of pinned staging buffers: a chunk's row tables are copied when the stream gets to them, which can be long after
        # the next chunk's tables are written on the host, so a buffer is refilled only once the copy that read it has run
        self.rows_ring = [torch.zeros(11 * T, dtype=torch.int32).pin_memory() for _ in range(3)]
        self.rows_events = [None] * 3
        self.rows_turn = 0
        self.rows_host = self.rows_ring[0]
        # KV spill: device copies of one slot's host pages of one layer; the attention of a chunk that reaches into the
        # spilled part reads them here instead of gathering rows over the host link (one lane only: the copy follows the
        # chunk's own key / value writes on the same stream)
        if dm.n_host_pages and st.spill_stage:
            spill = dm.max_pages - dm.dev_quota
            row = sc.kvh_l * c.head_dim
            self.b["stage_k"] = z((spill, DM.KV_PAGE, row), bf)
            self.b["stage_v"] = z((spill, DM.KV_PAGE, row), bf)
            self.lanes = 1
        self.side_stream = torch.cuda.Stream(device=dev) if self.lanes == 2 else None
        self.bufs = S.QwPrefillBufs()
        self._hook_cb = None
        self._over = None
        self._fill_struct()

    def _ensure_mtp_buffers(self):
        """Buffers of the MTP pass, made when a model with an MTP head first prefills."""
        if "Xm" in self.b:
            return
        dm, c, sc, T = self.dm, self.dm.cfg, self.dm.sc, self.T
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dm.dev)
        self.b["Xm"] = z((T, c.hc, sc.sh), torch.float32)
        self.b["hn"] = z((T * c.hc, c.hidden), torch.bfloat16) if not self.tp else None
        self.b["en"] = z((T, c.hidden), torch.bfloat16)
        self.b["fh"], self.b["fe"] = z((T * c.hc, sc.sh), torch.float32), z((T, sc.sh), torch.float32)
        self.b["mtp_ssq"] = z((2, T), torch.float32)
        self._fill_struct()

    def _fill_struct(self):
        b, s, T = self.b, self.bufs, self.T
        for name in S.PREFILL_PTR_FIELDS:
            t = b.get(name)
            setattr(s, name, None if t is None else t.data_ptr())
        r = b["rows"].data_ptr()
        s.tokens, s.slot, s.pos, s.run_start, s.run_len, s.ctx3 = r, r + 4 * T, r + 8 * T, r + 12 * T, r + 16 * T, r + 20 * T
        s.m_slot, s.m_pos, s.m_run_start, s.m_run_len, s.mtp_tok = r + 4 * T, r + 32 * T, r + 12 * T, r + 36 * T, r + 40 * T
        s.cap, s.hc_ld, s.hc_ksplit, s.nrs_ld, s.proj_ld = T, self.hc_ld, self.hc_ksplit, self.nrs_ld, self.proj_ld
        s.o_ld, s.ple_ld, s.max_tiles, s.gdn_scratch_lane = self.o_ld, self.ple_ld, self.max_tiles, self.gdn_scratch_lane

    # ---- helpers
    def _s(self):
        return P(torch.cuda.current_stream(self.dm.dev).cuda_stream)

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed: {rc}")

    def gemm(self, A, W_ptr, N, K, out, ldw=None):
        """out[:, :N] = A @ W^T with W given by pointer ([N][ldw] bf16)."""
        T = A.shape[0]
        self._ck(self.lib.qwk_gemm_bf16_tc(_p(A), P(W_ptr), _p(out), T, N, K, A.stride(0), ldw or K, out.stride(0),
                                           1 if out.dtype == torch.bfloat16 else 0, self._s()), "gemm")

    def lane_split(self, T: int):
        """Rows of lane 0 when a chunk of T rows runs as two micro-batches (a multiple of the GDN scan's 64-row chunk)."""
        if self.lanes < 2 or T < 2:
            return T
        n0 = (T // 2 + 63) // 64 * 64
        return n0 if n0 < T else T // 2

    def _rows(self, slot, base, T, toks, ctx3, mtp_tokens=(), mtp_base=0, n0=None):
        """Row tables of a chunk (pinned host memory -> device, one copy): tokens | slot | pos | run_start | run_len | ctx3 |
        MTP positions | MTP run_len | MTP next tokens.  Run tables are relative to a lane's first row."""
        Tm = self.T
        turn = self.rows_turn = (self.rows_turn + 1) % len(self.rows_ring)
        if self.rows_events[turn] is not None:
            self.rows_events[turn].synchronize()
        self.rows_host = self.rows_ring[turn]
        h = self.rows_host.numpy()
        h[0:T] = toks
        h[Tm:Tm + T] = slot
        h[2 * Tm:2 * Tm + T] = np.arange(base, base + T, dtype=np.int32)
        h[3 * Tm:3 * Tm + T] = 0
        h[4 * Tm:4 * Tm + T] = 0
        n0 = T if n0 is None else n0
        h[4 * Tm] = n0
        if n0 < T:
            h[4 * Tm + n0] = T - n0
        h[5 * Tm:5 * Tm + 3 * T] = ctx3.reshape(-1)
        nm = len(mtp_tokens)
        if nm:
            h[8 * Tm:8 * Tm + nm] = np.arange(mtp_base, mtp_base + nm, dtype=np.int32)
            h[9 * Tm:9 * Tm + nm] = 0
            h[9 * Tm] = nm
            h[10 * Tm:10 * Tm + nm] = mtp_tokens
        self.b["rows"].copy_(self.rows_host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.dm.dev))
        self.rows_events[turn] = ev
        r = self.b["rows"].data_ptr()
        return {"tokens": r, "slot": r + 4 * Tm, "pos": r + 8 * Tm, "run_start": r + 12 * Tm, "run_len": r + 16 * Tm,
                "ctx3": r + 20 * Tm}

    # ---- one chunk through the native runtime
    def make_job(self, slot: int, base: int, tokens: Sequence[int], ctx3: np.ndarray, want_logits: bool = True, embeds=None,
                 mtp: bool = False, pending: Optional[torch.Tensor] = None) -> S.QwPrefillJob:
        """Stage the chunk's row tables and describe it for ``qwrt_prefill``.  ``mtp``: also run the MTP head over the rows
        whose next token is known, preceded by the row of ``pending`` (the hidden state of the position before the chunk)."""
        dm, c = self.dm, self.dm.cfg
        T = len(tokens)
        assert 1 <= T <= self.T
        toks = [c.real_token(int(t)) for t in tokens]
        mtp_tokens, mtp_base = [], base
        if mtp:
            self._ensure_mtp_buffers()
            if pending is not None and base > 0:
                dm.buf["hidden_out"][0].copy_(pending)
                mtp_tokens, mtp_base = toks[:T], base - 1
            else:
                pending = None
                mtp_tokens = toks[1:T]
        lanes = self.lanes if T >= 128 else 1          # a short chunk runs as one lane
        n0 = self.lane_split(T) if lanes == 2 else T
        self._rows(slot, base, T, toks, np.asarray(ctx3, dtype=np.int32), mtp_tokens, mtp_base, n0)
        j = S.QwPrefillJob()
        j.md, j.b = C.pointer(dm.model), C.pointer(self.bufs)
        cur = torch.cuda.current_stream(dm.dev)
        j.stream[0] = cur.cuda_stream
        j.stream[1] = self.side_stream.cuda_stream if self.side_stream is not None else cur.cuda_stream
        for l in range(2):
            j.tp[l] = self.channels[min(l, len(self.channels) - 1)].ptr if self.tp else None
        j.T, j.lanes, j.base, j.want_logits = T, lanes, base, int(bool(want_logits))
        j.slot = int(slot)
        j.n0 = n0
        j.layer_limit = -1 if self.layer_limit is None else int(self.layer_limit)
        j.mtp_rows, j.mtp_base, j.has_pending = len(mtp_tokens), mtp_base, int(pending is not None)
        j.n_over = 0
        if embeds is not None:          # (row indices, [n, hidden] fp32): these rows' embedding replaces the table's
            rows_i, emb = embeds
            self._over = (rows_i.to(dm.dev, torch.int32).contiguous(), emb.to(dm.dev, torch.float32).contiguous())
            self.bufs.over_rows, self.bufs.over_emb = self._over[0].data_ptr(), self._over[1].data_ptr()
            j.n_over = int(self._over[0].numel())
        if self.on_block_input is not None:
            def hook(user, layer, which, bin_ptr, ld, r0, n):
                self.on_block_input(layer, "attn" if which == 0 else "mlp", self.block_input(0 if r0 == 0 else 1, r0, n))
            self._hook_cb = S.PREFILL_HOOK(hook)
            j.hook = self._hook_cb
        return j

    def block_input(self, lane: int, r0: int, n: int) -> torch.Tensor:
        """The block-input rows of a lane as a tensor [n, hidden] (bf16)."""
        H = self.dm.cfg.hidden
        if self.tp:
            return self.channels[lane].view(S.TP_BIN, n * H * 2, torch.bfloat16).view(n, H)
        return self.b["bin"][r0:r0 + n]

    @staticmethod
    def launch(lib, jobs: List[S.QwPrefillJob]) -> None:
        """Enqueue the chunk of every job (several jobs: emulated ranks of one process, all on one stream)."""
        arr = (C.POINTER(S.QwPrefillJob) * len(jobs))(*[C.pointer(j) for j in jobs])
        rc = lib.qwrt_prefill(arr, len(jobs))
        if rc != 0:
            raise RuntimeError(f"qwrt_prefill failed: {rc}")

    @torch.no_grad()
    def run(self, slot: int, base: int, tokens: Sequence[int], ctx3: np.ndarray, want_logits: bool = True, embeds=None,
            mtp: bool = False, pending: Optional[torch.Tensor] = None):
        """One chunk.  Returns the logits of the last token (this rank's vocabulary shard; the argmax over all ranks is in
        ``dm.buf['amax_idx'][0]``).  After a chunk with ``mtp``, ``self.b['hid_out']`` holds the next call's pending row."""
        if not self.native:
            return self.run_py(slot, base, tokens, ctx3, want_logits, embeds)
        job = self.make_job(slot, base, tokens, ctx3, want_logits, embeds, mtp, pending)
        self.launch(self.lib, [job])
        return self.dm.buf["logits"][0] if want_logits else None

    def mix(self, hc, T, pend, inj_prev, inj_out, n_inj):
        dm, b, c, sc, L = self.dm, self.b, self.dm.cfg, self.dm.sc, self.lib
        s = self._s()
        self._ck(L.qwk_hc_prenorm_T(_p(b["X"]), _p(pend), c.hidden, _p(inj_prev), P(hc["w1"].data_ptr()), sc.sh, c.hc,
                                    C.c_float(c.eps), _p(b["xn"]), T, s), "hc_prenorm")
        down = c.hc_rank + n_inj
        # few output tiles and a long K: the down projection runs split-K; hc_mid adds the partial sums in order
        ks = self.hc_ksplit
        self._ck(L.qwk_gemm_bf16_tc_splitk(_p(b["xn"]), P(hc["Wd"].data_ptr()), _p(b["d"]), T, down, c.hch, c.hch, c.hch,
                                           self.hc_ld, ks, self.T * self.hc_ld, s), "hc_down")
        self._ck(L.qwk_hc_mid_T(_p(b["d"]), self.hc_ld, c.hc_rank, n_inj, c.hc, _p(b["u"]), _p(inj_out), T, ks,
                                self.T * self.hc_ld, s), "hc_mid")
        self.gemm(b["u"][:T], hc["Wu"].data_ptr(), c.hch, c.hc_rank, b["g"][:T])
        self._ck(L.qwk_hc_mix_T(_p(b["g"]), _p(b["xn"]), sc.sh, _p(b["bin"]), c.hidden, T, s), "hc_mix")

    # ---- one chunk, scheduled from Python (one GPU, one lane)
    @torch.no_grad()
    def run_py(self, slot: int, base: int, tokens: Sequence[int], ctx3: np.ndarray, want_logits: bool = True, embeds=None):
        dm, b, c, sc, L = self.dm, self.b, self.dm.cfg, self.dm.sc, self.lib
        T = len(tokens)
        assert 1 <= T <= self.T and not self.tp
        s = self._s()
        rows = self._rows(slot, base, T, [c.real_token(int(t)) for t in tokens], np.asarray(ctx3, dtype=np.int32))
        self._last_rows = rows
        rp = lambda k, off=0: P(rows[k] + 4 * off)
        d = dm.model.d
        self._ck(L.qwk_embed_rows(rp("tokens"), P(dm.globals_w["embed"].data_ptr()), c.hidden, 0, sc.sh, c.hc, c.vocab,
                                  _p(b["X"]), T, s), "embed")
        if embeds is not None:          # (row indices, [n, hidden] fp32): these rows' embedding replaces the table's
            rows_i, emb = embeds
            X = b["X"][:T].view(T, c.hc, sc.sh)
            X[rows_i] = emb.to(X.dtype)[:, None, :sc.sh].expand(-1, c.hc, -1)
        pend, inj_prev = None, None
        inj_attn, inj_mlp = b["inj_a"], b["inj_b"]
        max_groups = (base + T) // c.idx_ratio
        for li in range(c.n_layers if self.layer_limit is None else min(c.n_layers, int(self.layer_limit))):
            lw = dm.layers_w[li]
            if li == c.ple_layer and dm.model.ple.enabled:
                if pend is not None:
                    self._ck(L.qwk_hc_pre(_p(b["X"]), _p(pend), c.hidden, _p(inj_prev), c.hc, None, sc.sh, c.hc, None, None, 0,
                                          T, s), "combine")
                    pend = None
                pw_ = dm.ple_w
                p = dm.model.ple
                self._ck(L.qwk_ple_gather(rp("ctx3"), P(p.shards), P(p.scales), p.rows_per_shard, p.rows, p.layout,
                                          c.ngram_dim, c.ngram_heads, _p(b["ple_e"]), None, T, s), "ple_gather")
                self.gemm(b["ple_e"][:T], pw_["Wkv"].data_ptr(), sc.ple_kv, c.hidden, b["ple_kv"][:T])
                ldk = b["ple_kv"].stride(0)
                self._ck(L.qwk_ple_stats(_p(b["ple_kv"]), ldk, _p(b["X"]), P(pw_["nk1"].data_ptr()), P(pw_["nq1"].data_ptr()),
                                         sc.sh, c.hc, _p(b["ple_send"]), 16, T, s), "ple_stats")
                self._ck(L.qwk_ple_apply(_p(b["ple_kv"]), ldk, _p(b["ple_send"]), 16, P(pw_["nc1"].data_ptr()),
                                         P(pw_["cw"].data_ptr()), sc.sh, c.hc, c.hidden, C.c_float(c.eps), c.ple_conv,
                                         c.ple_dilation, _p(b["ple_gv"]), _p(b["ple_nc"]), _p(dm.ple_ring), _p(b["X"]), T,
                                         rp("slot"), rp("pos"), rp("run_start"), rp("run_len"), s), "ple_apply")
            self.mix(lw["attn_hc"], T, pend, inj_prev, inj_attn, c.hc)
            if self.on_block_input is not None:
                self.on_block_input(li, "attn", b["bin"][:T])
            self.attn_block(lw, T, rp, max_groups, c.qsa_index(li) if lw["is_qsa"] else c.gdn_index(li))
            self.mix(lw["mlp_hc"], T, b["out_a"], inj_attn, inj_mlp, c.hc)
            if self.on_block_input is not None:
                self.on_block_input(li, "mlp", b["bin"][:T])
            self.moe(lw, T)
            pend, inj_prev = b["out_b"], inj_mlp
        gw = dm.globals_w
        self.mix(gw["final_hc"], T, pend, inj_prev, None, 0)
        if want_logits:
            last = b["bin"][T - 1:T]
            self._ck(L.qwk_gemv_bf16(P(gw["lm_head"].data_ptr()), _p(last), _p(dm.buf["logits"]), None, sc.vocab_l, c.hidden, 1,
                                     c.hidden, c.hidden, sc.vocab_l, 0, 1, 0, 0, 0, s), "lm_head")
            self._ck(L.qwk_row_reduce(_p(dm.buf["logits"]), sc.vocab_l, sc.vocab_l, 0, 1, _p(dm.buf["amax_val"]),
                                      _p(dm.buf["amax_idx"]), _p(dm.buf["lse_max"]), _p(dm.buf["lse_sum"]), s), "row_reduce")
        return dm.buf["logits"][0] if want_logits else None

    def attn_block(self, lw, T, rp, max_groups, state_index):
        """The attention block of one layer over T rows: bin -> out_a (fp32 [T][H])."""
        dm, b, c, sc, L = self.dm, self.b, self.dm.cfg, self.dm.sc, self.lib
        s = self._s()
        d = dm.model.d
        if lw["is_qsa"]:
            qi = state_index
            self.gemm(b["bin"][:T], lw["Wproj"].data_ptr(), sc.qsa_proj_l, c.hidden, b["proj"][:T])
            ldp = self.proj_ld
            kd, vd = dm.k_dev[qi].data_ptr(), dm.v_dev[qi].data_ptr()
            kh = dm.k_host[qi].data_ptr() if dm.k_host else None
            vh = dm.v_host[qi].data_ptr() if dm.v_host else None
            self._ck(L.qwk_qsa_prep(_p(b["proj"]), ldp, sc.qh_l, sc.kvh_l, c.idx_heads, P(lw["qn1"].data_ptr()),
                                    P(lw["kn1"].data_ptr()), P(lw["iqn1"].data_ptr()), P(lw["ikn1"].data_ptr()), T,
                                    rp("slot"), rp("pos"), rp("run_start"), rp("run_len"), P(kd), P(vd), P(kh) if kh else None,
                                    P(vh) if vh else None, d.n_dev_pages, _p(dm.page_table), d.max_pages, _p(b["q"]),
                                    _p(b["iq"]), _p(dm.raw_ring[qi]), _p(dm.ck[qi]), d.ck_cap, c.idx_ratio,
                                    C.c_float(c.eps), s), "qsa_prep")
            self._ck(L.qwk_qsa_scores(_p(b["iq"]), c.idx_heads, _p(dm.ck[qi]), d.ck_cap, T, rp("slot"), rp("pos"),
                                      c.idx_ratio, c.idx_topk_blocks, _p(b["scores"]), d.score_cap, max_groups, s), "scores")
            self._ck(L.qwk_qsa_select(_p(b["scores"]), d.score_cap, T, rp("pos"), c.idx_ratio, c.idx_topk_blocks,
                                      _p(b["sel"]), _p(b["sel_n"]), s), "select")
            ow = sc.qh_l * c.head_dim
            if self.qsa_mma:
                self._ck(L.qwk_qsa_attend_mma(_p(b["q"]), sc.qh_l, sc.kvh_l, T, rp("slot"), rp("pos"), P(kd), P(vd),
                                              P(kh) if kh else None, P(vh) if vh else None, d.n_dev_pages, _p(dm.page_table),
                                              d.max_pages, _p(b["sel"]), _p(b["sel_n"]), c.idx_topk_blocks, c.idx_ratio,
                                              _p(b["proj"]), ldp, _p(b["o"]), s), "attend_mma")
            else:
                A = self.attn_rows
                for r0 in range(0, T, A):
                    n = min(A, T - r0)
                    self._ck(L.qwk_qsa_attend(P(b["q"].data_ptr() + 4 * r0 * ow), sc.qh_l, sc.kvh_l, n, rp("slot", r0),
                                              rp("pos", r0), P(kd), P(vd), P(kh) if kh else None, P(vh) if vh else None,
                                              d.n_dev_pages, _p(dm.page_table), d.max_pages,
                                              P(b["sel"].data_ptr() + 4 * r0 * c.idx_topk_blocks),
                                              P(b["sel_n"].data_ptr() + 4 * r0), c.idx_topk_blocks, c.idx_ratio, d.nsplit,
                                              _p(b["pm"]), _p(b["pl"]), _p(b["pacc"]), P(b["proj"].data_ptr() + 4 * r0 * ldp),
                                              ldp, P(b["o"].data_ptr() + 2 * r0 * ow), s), "attend")
            # the attention kernels write o rows densely ([T][QL*256])
            self._ck(L.qwk_gemm_bf16_tc(_p(b["o"]), P(lw["Wout"].data_ptr()), _p(b["out_a"]), T, c.hidden, ow, ow, ow,
                                        c.hidden, 0, s), "o_proj")
        else:
            gi = state_index
            self.gemm(b["bin"][:T], lw["Wproj"].data_ptr(), sc.gdn_proj_l, c.hidden, b["proj"][:T])
            ldp = self.proj_ld
            self._ck(L.qwk_gdn_conv(_p(b["proj"]), ldp, _p(dm.gdn_ring[gi]), P(lw["cw"].data_ptr()), P(lw["A_log"].data_ptr()),
                                    P(lw["dt_bias"].data_ptr()), sc.gdn_kl, sc.gdn_vl, T, rp("slot"), rp("pos"),
                                    rp("run_start"), rp("run_len"), _p(b["qkv"]), _p(b["decay"]), _p(b["beta"]),
                                    C.c_float(c.eps), s), "gdn_conv")
            if self.gdn_chunked:
                self._ck(L.qwk_gdn_scan_chunked(_p(b["qkv"]), _p(b["decay"]), _p(b["beta"]), _p(b["proj"]), ldp,
                                                _p(dm.gdn_S[gi]), P(lw["gdn_norm"].data_ptr()), sc.gdn_kl, sc.gdn_vl, T,
                                                rp("slot"), _p(b["gdn_scratch"]), _p(b["o"]), C.c_float(c.eps), s),
                         "gdn_scan_chunked")
            else:
                self._ck(L.qwk_gdn_scan(_p(b["qkv"]), _p(b["decay"]), _p(b["beta"]), _p(b["proj"]), ldp, _p(dm.gdn_S[gi]), None,
                                        P(lw["gdn_norm"].data_ptr()), sc.gdn_kl, sc.gdn_vl, T, rp("slot"), rp("pos"),
                                        rp("run_start"), rp("run_len"), _p(b["o"]), C.c_float(c.eps), s), "gdn_scan")
            ow = sc.gdn_vl * c.gdn_dim
            # gdn_scan writes o rows densely ([T][VL*128])
            self._ck(L.qwk_gemm_bf16_tc(_p(b["o"]), P(lw["Wout"].data_ptr()), _p(b["out_a"]), T, c.hidden, ow, ow, ow,
                                        c.hidden, 0, s), "gdn_out")

    def mtp_pass(self, slot: int, base: int, T: int, next_tokens, keep_last_hidden: bool = True):
        """MTP rows for positions base..base+T-1 whose hidden states are in X (after run()) and whose next
        tokens are ``next_tokens`` (the last position's may be missing: it is handled when the token is known)."""
        dm, b, c, sc, L = self.dm, self.b, self.dm.cfg, self.dm.sc, self.lib
        w = dm.mtp_w
        n = len(next_tokens)
        if n == 0:
            return
        s = self._s()
        self._ensure_mtp_buffers()
        if "mtp_tok_py" not in b:
            b["mtp_tok_py"] = torch.zeros((self.T,), dtype=torch.int32, device=dm.dev)
        b["mtp_tok_py"][:n].copy_(torch.as_tensor([c.real_token(int(t)) for t in next_tokens], dtype=torch.int32), non_blocking=True)
        rows = self._last_rows
        rp = lambda k, off=0: P(rows[k] + 4 * off)
        self._ck(L.qwk_mtp_norm(_p(b["X"]), _p(b["mtp_tok_py"]), P(dm.globals_w["embed"].data_ptr()), c.vocab, P(w["nh1"].data_ptr()),
                                P(w["ne1"].data_ptr()), c.hidden, c.hc, C.c_float(c.eps), _p(b["hn"]), _p(b["en"]), n, s), "mtp_norm")
        self.gemm(b["hn"][:n * c.hc], w["fc_h"].data_ptr(), c.hidden, c.hidden, b["fh"][:n * c.hc])
        self.gemm(b["en"][:n], w["fc_e"].data_ptr(), c.hidden, c.hidden, b["fe"][:n])
        self._ck(L.qwk_mtp_add(_p(b["fh"]), _p(b["fe"]), c.hidden, c.hc, _p(b["X"]), n, s), "mtp_add")
        lw = w["layer"]
        self.mix(lw["attn_hc"], n, None, None, b["inj_a"], c.hc)
        self.attn_block(lw, n, rp, (base + n) // c.idx_ratio, c.n_qsa)
        self.mix(lw["mlp_hc"], n, b["out_a"], b["inj_a"], b["inj_b"], c.hc)
        self.moe(lw, n)
        # the MTP layer's output is not needed for prompt rows: only its KV / indexer state matters

    def moe(self, lw, T):
        dm, b, c, sc, L = self.dm, self.b, self.dm.cfg, self.dm.sc, self.lib
        s = self._s()
        E, k, F, H = sc.exp_l, c.top_k, c.ffn, c.hidden
        nrs = c.n_experts + 1 + 2 * sc.sffn_l
        self.gemm(b["bin"][:T], lw["Wrs"].data_ptr(), nrs, H, b["rs"][:T])
        self._ck(L.qwk_moe_route(_p(b["rs"]), self.nrs_ld, T, c.n_experts, k, sc.sffn_l, 0, E, _p(b["pe"]), _p(b["pw"]),
                                 _p(b["sh_h"]), s), "route")
        # ---- expert sort: pairs of one expert become consecutive rows; tile tables for the grouped GEMMs; row gather
        Pn = T * k
        inv, t13, t2 = b["inv"], b["t13"], b["t2"]
        self._ck(L.qwk_moe_sort_T(_p(b["pe"]), T, k, E, 2 * F, H, self.max_tiles, _p(inv), _p(b["src_token"]), _p(t13), _p(t2),
                                  _p(b["bin"]), b["bin"].stride(0), H, _p(b["xperm"]), s), "moe_sort")
        if self.q4_fused:
            # q4 words converted inside the GEMM's W-operand producer warps: no bf16 copy of the layer's experts
            self._ck(L.qwk_gemm_q4_tc_grouped(_p(b["xperm"]), P(lw["w13"].data_ptr()), P(lw["s13"].data_ptr()), _p(b["h13"]),
                                              _p(t13), self.max_tiles, Pn, E * 2 * F, 2 * F, H, H, 2 * F, 1, s), "experts13")
            self._ck(L.qwk_swiglu_T(_p(b["h13"]), F, _p(b["h"]), Pn, s), "swiglu")
            self._ck(L.qwk_gemm_q4_tc_grouped(_p(b["h"]), P(lw["w2"].data_ptr()), P(lw["s2"].data_ptr()), _p(b["y"]), _p(t2),
                                              self.max_tiles, Pn, E * H, H, F, F, H, 0, s), "experts2")
        else:
            self._ck(L.qwk_q4_dequant(P(lw["w13"].data_ptr()), P(lw["s13"].data_ptr()), E * 2 * F, H, _p(b["w13dq"]), s), "dequant13")
            self._ck(L.qwk_q4_dequant(P(lw["w2"].data_ptr()), P(lw["s2"].data_ptr()), E * H, F, _p(b["w2dq"]), s), "dequant2")
            self._ck(L.qwk_gemm_bf16_tc_grouped(_p(b["xperm"]), _p(b["w13dq"]), _p(b["h13"]), _p(t13), self.max_tiles, Pn,
                                                E * 2 * F, 2 * F, H, H, H, 2 * F, 1, s), "experts13")
            self._ck(L.qwk_swiglu_T(_p(b["h13"]), F, _p(b["h"]), Pn, s), "swiglu")
            self._ck(L.qwk_gemm_bf16_tc_grouped(_p(b["h"]), _p(b["w2dq"]), _p(b["y"]), _p(t2), self.max_tiles, Pn, E * H, H, F, F,
                                                F, H, 0, s), "experts2")
        self.gemm(b["sh_h"][:T], lw["Wsd"].data_ptr(), H, sc.sffn_l, b["sd"][:T])
        self._ck(L.qwk_moe_combine_T(_p(b["y"]), H, _p(inv), _p(b["pw"]), k, _p(b["sd"]), H, _p(b["out_b"]), T, s), "combine")
