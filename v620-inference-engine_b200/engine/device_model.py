"""One rank's model on the device: engine-layout weights, slot state, work buffers and the
ctypes structs handed to the native runtime (``qwrt_decode``).

PyTorch owns every allocation; the runtime only enqueues kernels.  A step of ``M`` rows is either
launched directly or replayed from a CUDA graph captured per row count (reference:
``launch_graph``, src/engine/decode.hip:166-181, captures one graph per M and kind).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import ModelConfig, ShardConfig
from ..models.ngram import NgramHasher
from ..models.ple import PleTable, f8e4m3_lut
from ..models.weights import Weights
from ..ops import lib as qlib
from ..ops import structs as S
from . import weights_prep as WP

KV_PAGE = 256
RAW_RING = 16
GDN_RING = 16
PLE_RING = 32
MAX_ROWS = 32
def gpu_numa_node(dev) -> int:
    """NUMA node of the GPU's PCI function (sysfs), -1 when the system does not say."""
    try:
        props = torch.cuda.get_device_properties(dev)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            return int(f.read().strip())
    except Exception:          # noqa: BLE001 - no sysfs entry, no CUDA device, a property this torch lacks
        return -1


_SPILL_KEEPALIVE: list = []      # spill-cache buffers of every model made in this process (see _alloc_spill_cache)
PLE_LAYOUT_ID = {"f8": 0, "bf16": 1, "int8": 2, "int4": 3}

FLAG_SAVE_GDN = 1
FLAG_NO_HEAD = 2
FLAG_KEEP_HIDDEN = 4
FLAG_CHAIN = 8


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class DeviceModel:
    def __init__(self, cfg: ModelConfig, ranks: int = 1, rank: int = 0, device: str = "cuda:0", slots: int = 1,
                 slot_tokens: int = 8192, max_rows: int = MAX_ROWS, host_pages: int = 0,
                 dev_pages: Optional[int] = None, save_gdn: bool = False):
        self.cfg, self.sc = cfg, ShardConfig(cfg, ranks, rank)
        self.dev = torch.device(device)
        self.slots, self.max_rows = slots, max_rows
        self.slot_tokens = int(math.ceil(slot_tokens / KV_PAGE) * KV_PAGE)
        self.max_pages = self.slot_tokens // KV_PAGE
        self.n_dev_pages = dev_pages if dev_pages is not None else slots * self.max_pages
        self.n_host_pages = host_pages
        self.lib = qlib.load(required=True)
        self.keep: List[object] = []          # tensors referenced by raw pointers
        self.layers_w: List[Dict[str, object]] = []
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.model = S.QwModel()
        self._layers_arr = (S.QwLayer * cfg.n_layers)()
        self.model.layers = C.cast(self._layers_arr, C.POINTER(S.QwLayer))
        from ..utils import settings as _settings
        self.guard_on = bool(_settings.get().guard)
        self.guards: Dict[str, torch.Tensor] = {}
        self._guard_raw = []
        self.steps_run = 0
        self._fill_dims()
        self._alloc_state()
        self._alloc_spill_cache(int(_settings.get().spill_cache_mb), bool(_settings.get().spill_cache_stats))
        self._alloc_buffers(save_gdn)
        self._alloc_rows()
        qlib.check(self.lib.qwk_rope_init(C.c_double(cfg.rope_theta), cfg.rope_dim), "rope_init")
        # error word for kernels with bounded waits: (code, detail), 0 = ok
        self.err_word = torch.zeros(2, dtype=torch.int32, device=self.dev)
        self.moe_stats = None
        if _settings.get().moe_stats:           # QW_MOE_STATS: per-layer count of expert pairs computed on this rank
            self.moe_stats = torch.zeros(cfg.n_layers + 1, dtype=torch.int32, device=self.dev)
            self.lib.qwrt_set_moe_stats(C.c_void_p(self.moe_stats.data_ptr()))
        self.lib.qwk_set_error_word(C.c_void_p(self.err_word.data_ptr()))
        self._init_ngram()
        self.comm_cb = None

    # ------------------------------------------------------------------ dims
    def _fill_dims(self):
        c, sc, d = self.cfg, self.sc, self.model.d
        d.ranks, d.rank = sc.ranks, sc.rank
        d.H, d.hc, d.hc_rank, d.SH = c.hidden, c.hc, c.hc_rank, sc.sh
        d.n_layers, d.vocab, d.vocab_l = c.n_layers, c.vocab, sc.vocab_l
        d.QL, d.KVL, d.IH, d.proj_qsa = sc.qh_l, sc.kvh_l, c.idx_heads, sc.qsa_proj_l
        d.KL, d.VL, d.proj_gdn = sc.gdn_kl, sc.gdn_vl, sc.gdn_proj_l
        d.E, d.E_l, d.e_first, d.top_k, d.F, d.SF = c.n_experts, sc.exp_l, sc.rank * sc.exp_l, c.top_k, c.ffn, sc.sffn_l
        d.ple_layer, d.ple_kv, d.ngram_heads, d.ngram_dim = c.ple_layer, sc.ple_kv, c.ngram_heads, c.ngram_dim
        d.ple_taps, d.ple_dil = c.ple_conv, c.ple_dilation
        d.idx_ratio, d.idx_topk = c.idx_ratio, c.idx_topk_blocks
        d.nsplit = (c.idx_budget + c.idx_ratio + 63) // 64
        d.max_rows = self.max_rows
        d.slots, d.max_pages, d.n_dev_pages = self.slots, self.max_pages, self.n_dev_pages
        d.ck_cap = self.slot_tokens // c.idx_ratio
        d.score_cap = d.ck_cap
        d.eps = c.eps
        assert c.gdn_dim == 128 and c.head_dim == 256 and c.idx_dim == 128 and c.hc == 4

    # ------------------------------------------------------------------ state
    def _alloc_state(self):
        c, sc, dv = self.cfg, self.sc, self.dev
        row = sc.kvh_l * c.head_dim
        nkv = c.n_qsa + (1 if c.mtp else 0)      # the MTP layer keeps its own KV / indexer state at index n_qsa
        z = lambda *shape, dtype=torch.float32: torch.zeros(*shape, dtype=dtype, device=dv)
        self.k_dev = [z(self.n_dev_pages, KV_PAGE, row, dtype=torch.bfloat16) for _ in range(nkv)]
        self.v_dev = [z(self.n_dev_pages, KV_PAGE, row, dtype=torch.bfloat16) for _ in range(nkv)]
        self.k_host = self.v_host = None
        self.spill_numa = None
        if self.n_host_pages:
            self.k_host, self.v_host = self._alloc_spill_pool(nkv, row)
        self.ck = [z(self.slots, self.slot_tokens // c.idx_ratio, c.idx_dim, dtype=torch.bfloat16) for _ in range(nkv)]
        self.raw_ring = [z(self.slots, RAW_RING, c.idx_dim) for _ in range(nkv)]
        self.gdn_S = [z(self.slots, sc.gdn_vl, c.gdn_dim, c.gdn_dim) for _ in range(c.n_gdn)]
        self.gdn_ring = [z(self.slots, GDN_RING, sc.gdn_qkv_l) for _ in range(c.n_gdn)]
        self.ple_ring = z(self.slots, PLE_RING, sc.xw)
        # Paging.  Everything on the device: slot s owns pages [s*max_pages, (s+1)*max_pages).  With a smaller
        # device pool every slot keeps its first `quota` pages in HBM and the rest of its pages live in the
        # pinned host pool (KV spill): page ids >= n_dev_pages address host memory, which the kernels read directly.
        total = self.slots * self.max_pages
        if self.n_dev_pages >= total:
            pt = torch.arange(total, dtype=torch.int32).view(self.slots, self.max_pages)
            self.dev_quota = self.max_pages
        else:
            quota = self.n_dev_pages // self.slots
            spill = self.max_pages - quota
            if self.n_host_pages < self.slots * spill:
                raise ValueError("host_pages too small for the requested KV spill")
            pt = torch.empty((self.slots, self.max_pages), dtype=torch.int32)
            for s_ in range(self.slots):
                pt[s_, :quota] = torch.arange(s_ * quota, (s_ + 1) * quota)
                pt[s_, quota:] = self.n_dev_pages + torch.arange(s_ * spill, (s_ + 1) * spill)
            self.dev_quota = quota
        self.page_table_host = pt.clone()
        self.page_table = pt.to(dv)
        st = self.model.st

        def parr(ts):
            a = (C.c_void_p * max(1, len(ts)))(*[t.data_ptr() for t in ts])
            self.keep.append(a)
            return C.cast(a, C.c_void_p)
        st.k_dev, st.v_dev = parr(self.k_dev), parr(self.v_dev)
        st.k_host = parr(self.k_host) if self.k_host else None
        st.v_host = parr(self.v_host) if self.v_host else None
        st.ck, st.raw_ring = parr(self.ck), parr(self.raw_ring)
        st.gdn_S, st.gdn_ring = parr(self.gdn_S), parr(self.gdn_ring)
        st.ple_ring = self.ple_ring.data_ptr()
        st.page_table = self.page_table.data_ptr()

    def reset_slot(self, slot: int):
        for t in self.gdn_S + self.gdn_ring + self.raw_ring:
            t[slot].zero_()
        self.ple_ring[slot].zero_()

    # ------------------------------------------------------------------ cache of host KV rows
    def _alloc_spill_pool(self, nkv: int, row: int):
        """Host pages of the KV spill: pinned memory the kernels address directly.  With a NUMA policy other than
        ``process`` (setting ``spill_policy``: auto = bind to the GPU's node when the machine has several) the pages
        come from one arena of the pinned pool - mmap, mbind, touch, register - and the node they landed on is read back
        (``spill_numa``); otherwise, or when that fails, from the CUDA allocator under the process's own policy.
        (reference: src/engine/spill.cpp:64-164)"""
        from ..native import host as H
        from ..utils import settings as _settings
        per = self.n_host_pages * KV_PAGE * row * 2
        pol = _settings.get().spill_policy
        node = gpu_numa_node(self.dev)
        try:
            nodes = H.numa_nodes()
        except Exception:
            nodes = 1
        if pol == "auto":
            pol = "bind" if (nodes > 1 and node >= 0) else "process"
        if pol != "process":
            try:
                unit = (per + 4095) // 4096 * 4096
                pool = H.PinnedPool(unit_bytes=unit, arena_bytes=unit * 2 * nkv, standing_units=0, use_cuda=True, policy=pol, node=node)
                pool.reserve(2 * nkv)
                views = [pool.get() for _ in range(2 * nkv)]
                ts = [torch.from_numpy(v[:per]).view(torch.bfloat16).view(self.n_host_pages, KV_PAGE, row) for v in views]
                for t in ts:
                    t.zero_()
                st = pool.stats()
                if not st["cuda_registered"]:
                    raise RuntimeError("the arena could not be registered with CUDA")
                self._spill_pool, self._spill_views = pool, views          # the pool owns the memory for the model's lifetime
                self.spill_numa = {"policy": pol, "node_wanted": node, "node_got": st["numa_node"], "nodes": nodes}
                return ts[:nkv], ts[nkv:]
            except Exception as ex:          # noqa: BLE001 - placement is an optimisation: fall back and say so
                self.spill_numa = {"policy": "process", "fallback": str(ex)[:120]}
        hp = lambda: torch.zeros(self.n_host_pages, KV_PAGE, row, dtype=torch.bfloat16).pin_memory()
        if self.spill_numa is None:
            self.spill_numa = {"policy": "process", "nodes": nodes}
        return [hp() for _ in range(nkv)], [hp() for _ in range(nkv)]

    def _alloc_spill_cache(self, mb: int, stats: bool):
        """Direct-mapped device cache in front of the pinned host KV pages (one entry = K row + V row of one token of
        one layer; reference: SpillCache in src/kernels/types.hpp:48-70, sized by QW_SPILL_CACHE_MB).  The kernels
        find it through a process-wide pointer set, so the newest model with host pages owns it; the buffers of
        earlier models stay referenced, because captured graphs of theirs may still name them."""
        self.spill_cache = None
        if not self.n_host_pages or mb <= 0:
            self.lib.qwk_set_spill_cache(None, None, None, None, None, 0, 0)
            return
        row = self.sc.kvh_l * self.cfg.head_dim
        entries = 1
        while entries * 2 * (4 * row + 8) <= mb << 20:
            entries *= 2
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=self.dev)
        sc_ = {"tags": z(entries, torch.int64), "rows": z(entries * 2 * row, torch.bfloat16), "miss": z(1 << 16, torch.int64),
               "ctl": z(2, torch.int32), "stats": z(2, torch.int64) if stats else None, "entries": entries}
        rc = self.lib.qwk_set_spill_cache(sc_["tags"].data_ptr(), sc_["rows"].data_ptr(), sc_["miss"].data_ptr(), sc_["ctl"].data_ptr(),
                                          sc_["stats"].data_ptr() if stats else None, entries, 1 << 16)
        if rc != 0:
            raise RuntimeError(f"qwk_set_spill_cache failed: {rc}")
        self.spill_cache = sc_
        _SPILL_KEEPALIVE.append(sc_)

    def spill_cache_clear(self):
        """Forget every cached row: for writers of host pages that are not kernels of the step (state import, slot copy)."""
        if self.spill_cache is not None:
            self.spill_cache["tags"].zero_()
            self.spill_cache["ctl"].zero_()

    def spill_cache_stats(self):
        """(hits, misses) of host-row reads since the model was made; None without QW_SPILL_CACHE_STATS."""
        if self.spill_cache is None or self.spill_cache["stats"] is None:
            return None
        h, m = self.spill_cache["stats"].tolist()
        return int(h), int(m)

    # ------------------------------------------------------------------ buffers
    def _alloc_buffers(self, save_gdn: bool):
        c, sc, dv, R = self.cfg, self.sc, self.dev, self.max_rows
        d = self.model.d
        f32, bf, i32 = torch.float32, torch.bfloat16, torch.int32
        hc_send = sc.hc_send
        shapes = {
            "X": ((R, c.hc, sc.sh), f32), "y": ((R, c.hc, sc.sh), bf), "send": ((R, hc_send), f32),
            "red": ((R, hc_send), f32), "bin": ((R, c.hidden), bf),
            "proj": ((R, max(sc.gdn_proj_l, sc.qsa_proj_l)), f32), "inj_a": ((R, c.hc), f32), "inj_b": ((R, c.hc), f32),
            "partial": ((R, c.hidden), f32), "out_a": ((R, sc.sh), f32), "out_b": ((R, sc.sh), f32),
            "o": ((R, max(sc.gdn_vl * c.gdn_dim, sc.qh_l * c.head_dim)), bf),
            "qkv": ((R, sc.gdn_qkv_l), f32), "decay": ((R, sc.gdn_vl), f32), "beta": ((R, sc.gdn_vl), f32),
            "q": ((R, sc.qh_l, c.head_dim), f32), "iq": ((R, c.idx_heads, c.idx_dim), f32),
            "scores": ((R, d.score_cap), f32), "sel": ((R, c.idx_topk_blocks), i32), "sel_n": ((R,), i32),
            "pm": ((R, sc.qh_l, d.nsplit), f32), "pl": ((R, sc.qh_l, d.nsplit), f32),
            "pacc": ((R, sc.qh_l, d.nsplit, c.head_dim), f32),
            "rs": ((R, c.n_experts + 1 + 2 * sc.sffn_l), f32), "pair_expert": ((R, c.top_k), i32),
            "pair_w": ((R, c.top_k), f32), "sh_h": ((R, sc.sffn_l), bf), "moe_h": ((R * c.top_k, c.ffn), bf),
            "ple_e": ((R, c.hidden), bf), "ple_kv": ((R, sc.ple_kv), f32), "ple_send": ((R, 16), f32),
            "ple_red": ((R, 16), f32), "ple_gv": ((R, sc.xw), f32), "ple_nc": ((R, sc.xw), f32),
            "logits": ((R, sc.vocab_l), f32), "amax_val": ((R,), f32), "amax_idx": ((R,), i32),
            "lse_max": ((R,), f32), "lse_sum": ((R,), f32), "hidden_out": ((R, c.hc, sc.sh), f32),
            "X2": ((R, c.hc, sc.sh), f32), "ticket": ((4,), i32),
        }
        if save_gdn:
            shapes["gdn_save"] = ((c.n_gdn, R, sc.gdn_vl, c.gdn_dim, c.gdn_dim), f32)
        self.buf: Dict[str, torch.Tensor] = {}
        for name in S.BUFFER_FIELDS:
            if name in shapes:
                shp, dt = shapes[name]
                self.buf[name] = self._zeros(name, shp, dt)
                setattr(self.model.b, name, self.buf[name].data_ptr())
            else:
                setattr(self.model.b, name, None)

    def _alloc_rows(self):
        R = self.max_rows
        # ring of pinned staging buffers: a buffer is refilled only after the copy that read it has run
        self.rows_ring = [torch.zeros(8 * R, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.rows_events = [None] * 4
        self.rows_turn = 0
        self.rows_host = self.rows_ring[0]
        self.rows_dev = torch.zeros(8 * R, dtype=torch.int32, device=self.dev)
        self.rows = S.QwRows()
        base = self.rows_dev.data_ptr()
        self.rows.tokens = base
        self.rows.slot = base + 4 * R
        self.rows.pos = base + 8 * R
        self.rows.run_start = base + 12 * R
        self.rows.run_len = base + 16 * R
        self.rows.ctx3 = base + 20 * R

    def _init_ngram(self):
        h = NgramHasher(self.cfg)
        self.hasher = h
        mult = (C.c_ulonglong * 4)(*(h.mult + [0] * (4 - len(h.mult))))
        sizes = (C.c_ulonglong * len(h.sizes))(*h.sizes)
        offs = (C.c_longlong * len(h.offsets))(*h.offsets)
        self._f8_lut = None
        qlib.check(self.lib.qwk_ple_init(C.cast(mult, C.c_void_p), self.cfg.ngram, C.cast(sizes, C.c_void_p),
                                         C.cast(offs, C.c_void_p), self.cfg.ngram_heads, self.cfg.eos, None), "ple_init")
        self.model.ple.enabled = 0

    # ------------------------------------------------------------------ weights
    def _hc_struct(self, hc: Dict[str, object]) -> S.QwHc:
        s = S.QwHc()
        s.w1, s.Wd, s.Wu, s.n_inj = hc["w1"].data_ptr(), hc["Wd"].data_ptr(), hc["Wu"].data_ptr(), int(hc["n_inj"])
        return s

    def _cached(self, name: str, make):
        """The converted tensors of one loading step: from the weight cache when it is replaying, else made now (and
        recorded when a cache is attached).  ``self.weight_cache`` is set by ``Engine.from_checkpoint``."""
        wc = getattr(self, "weight_cache", None)
        if wc is not None and wc.replaying:
            return wc.get(name, self.dev)
        obj = make()
        if wc is not None:
            wc.put(name, obj)
        return obj

    def set_layer(self, L: int, w: Optional[Weights]):
        """Install decoder layer ``L`` from checkpoint-named tensors (any device; None when the weight cache replays)."""
        lw = self._cached(f"layer{L}", lambda: WP.prep_layer(self.cfg, w, L, self.sc, self.dev))
        self.layers_w.append(lw)
        st = self._layers_arr[L]
        st.is_qsa = 1 if lw["is_qsa"] else 0
        st.state_index = self.cfg.qsa_index(L) if lw["is_qsa"] else self.cfg.gdn_index(L)
        st.attn_hc, st.mlp_hc = self._hc_struct(lw["attn_hc"]), self._hc_struct(lw["mlp_hc"])
        for k in ("Wproj", "Wout", "Wrs", "w13", "s13", "w2", "s2", "Wsd"):
            setattr(st, k, lw[k].data_ptr())
        for k in ("cw", "A_log", "dt_bias", "gdn_norm", "qn1", "kn1", "iqn1", "ikn1"):
            setattr(st, k, lw[k].data_ptr() if k in lw else None)
        if L == self.cfg.ple_layer:
            has = w is not None and f"layers.{L}.ple.key_proj.weight" in w
            pw = self._cached("ple", lambda: WP.prep_ple(self.cfg, w, self.sc, self.dev) if has else {})
            if not pw:
                return
            self.ple_w = pw
            p = self.model.ple
            for k in ("Wkv", "nk1", "nq1", "nc1", "cw"):
                setattr(p, k, pw[k].data_ptr())

    def _layer_struct(self, st, lw, state_index: int):
        st.is_qsa = 1 if lw["is_qsa"] else 0
        st.state_index = state_index
        st.attn_hc, st.mlp_hc = self._hc_struct(lw["attn_hc"]), self._hc_struct(lw["mlp_hc"])
        for k in ("Wproj", "Wout", "Wrs", "w13", "s13", "w2", "s2", "Wsd"):
            setattr(st, k, lw[k].data_ptr())
        for k in ("cw", "A_log", "dt_bias", "gdn_norm", "qn1", "kn1", "iqn1", "ikn1"):
            setattr(st, k, lw[k].data_ptr() if k in lw else None)

    def set_mtp(self, w: Weights):
        """Install the MTP head (a QSA decoder layer with its own mixer, the two fc matrices and norms)."""
        c, sc, dv = self.cfg, self.sc, self.dev
        cols = sc.cols()          # the fc matrices are sliced by output rows: their products are this rank's residual columns
        conv = self._cached("mtp", lambda: {
            "layer": WP.prep_layer(c, w, c.n_layers, sc, dv, prefix="mtp.layers.0.", qsa=True),
            "final_hc": WP.prep_hc(w, "mtp.hyper_connection_mixer.", sc, False, dv),
            "fc_h": w["mtp.fc_hidden.weight"].to(dv)[cols].to(torch.bfloat16).contiguous(),
            "fc_e": w["mtp.fc_embedding.weight"].to(dv)[cols].to(torch.bfloat16).contiguous(),
            "nh1": (1.0 + w["mtp.pre_fc_norm_hidden.weight"].to(dv).float()).contiguous(),
            "ne1": (1.0 + w["mtp.pre_fc_norm_embedding.weight"].to(dv).float()).contiguous()})
        lw, fin = conv["layer"], conv["final_hc"]
        R = self.max_rows
        m = self.model.mtp
        self.mtp_w = {
            **conv,
            "hn": torch.zeros((R * c.hc, c.hidden), dtype=torch.bfloat16, device=dv),
            "en": torch.zeros((R, c.hidden), dtype=torch.bfloat16, device=dv),
            "fh": torch.zeros((R * c.hc, sc.sh), dtype=torch.float32, device=dv),
            "fe": torch.zeros((R, sc.sh), dtype=torch.float32, device=dv),
        }
        self._layer_struct(m.layer, lw, c.n_qsa)
        m.final_hc = self._hc_struct(fin)
        for k in ("fc_h", "fc_e", "nh1", "ne1", "hn", "en", "fh", "fe"):
            setattr(m, k, self.mtp_w[k].data_ptr())
        m.enabled = 1

    def launch_mtp(self, flags: int = 0):
        s = torch.cuda.current_stream(self.dev).cuda_stream
        rc = self.lib.qwrt_mtp(C.byref(self.model), C.byref(self.rows), flags, C.c_void_p(s))
        if rc != 0:
            raise RuntimeError(f"qwrt_mtp failed: {rc}")

    def mtp_step(self, tokens, slots, pos, flags: int = 0, graph: bool = False):
        """One MTP pass: buf['hidden_out'] holds the rows' hidden states, ``tokens`` the tokens after them."""
        self.stage_rows(tokens, slots, pos, None)
        if not graph:
            self.launch_mtp(flags)
            return
        key = ("mtp", len(tokens), flags)
        g = self.graphs.get(key)
        if g is None:
            self.rows.max_groups = self.model.d.ck_cap
            self.launch_mtp(flags)
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.launch_mtp(flags)
            self.graphs[key] = g
            return
        g.replay()

    def set_globals(self, w: Weights):
        g = self._cached("globals", lambda: WP.prep_globals(self.cfg, w, self.sc, self.dev))
        self.globals_w = g
        self.model.embed = g["embed"].data_ptr()
        self.model.lm_head = g["lm_head"].data_ptr()
        self.model.final_hc = self._hc_struct(g["final_hc"])

    def set_ple_table(self, table: PleTable, to_device: bool = False):
        """Attach the n-gram table.  Shards stay where they are (pinned host memory is read by the
        gather kernel directly) unless ``to_device`` copies them to the GPU."""
        key = {"f8": "weight_f8", "bf16": "weight", "int8": "weight_i8", "int4": "weight_i4"}[table.layout]
        vals, scs = [], []
        for sh in table.shards:
            v = sh[key]
            if to_device or not (v.is_pinned() or v.is_cuda):
                v = v.to(self.dev)
            vals.append(v)
            if "weight_scale" in sh:
                s_ = sh["weight_scale"]
                if to_device or not (s_.is_pinned() or s_.is_cuda):
                    s_ = s_.to(self.dev)
                scs.append(s_)
        self.keep += vals + scs
        self.ple_ptrs = torch.tensor([v.data_ptr() for v in vals], dtype=torch.int64, device=self.dev)
        self.ple_sptrs = torch.tensor([s_.data_ptr() for s_ in scs] or [0], dtype=torch.int64, device=self.dev)
        p = self.model.ple
        p.shards, p.scales = self.ple_ptrs.data_ptr(), self.ple_sptrs.data_ptr()
        p.rows_per_shard, p.rows = table.rows_per_shard, table.rows
        p.layout, p.enabled = PLE_LAYOUT_ID[table.layout], 1
        if table.layout == "f8":
            lut = f8e4m3_lut(table.scale).contiguous()
            h = NgramHasher(self.cfg)
            mult = (C.c_ulonglong * 4)(*(h.mult + [0] * (4 - len(h.mult))))
            sizes = (C.c_ulonglong * len(h.sizes))(*h.sizes)
            offs = (C.c_longlong * len(h.offsets))(*h.offsets)
            qlib.check(self.lib.qwk_ple_init(C.cast(mult, C.c_void_p), self.cfg.ngram, C.cast(sizes, C.c_void_p),
                                             C.cast(offs, C.c_void_p), self.cfg.ngram_heads, self.cfg.eos,
                                             C.c_void_p(lut.data_ptr())), "ple_init")
        self.table = table

    def load_weights(self, layer_fn: Callable[[int], Weights], globals_w: Weights):
        self.set_globals(globals_w)
        for L in range(self.cfg.n_layers):
            self.set_layer(L, layer_fn(L))

    def weight_bytes(self) -> int:
        n = 0
        def walk(o):
            nonlocal n
            if isinstance(o, torch.Tensor):
                n += o.numel() * o.element_size()
            elif isinstance(o, dict):
                for v in o.values():
                    walk(v)
        for lw in self.layers_w:
            walk(lw)
        walk(getattr(self, "globals_w", {}))
        walk(getattr(self, "ple_w", {}))
        return n

    # ------------------------------------------------------------------ stepping
    def stage_rows(self, tokens: Sequence[int], slots: Sequence[int], pos: Sequence[int],
                   ctx3: Optional[np.ndarray] = None):
        """Fill the row tables (pinned host) and enqueue their copy to the device."""
        M, R = len(tokens), self.max_rows
        assert 1 <= M <= R
        turn = self.rows_turn = (self.rows_turn + 1) % len(self.rows_ring)
        if self.rows_events[turn] is not None:
            self.rows_events[turn].synchronize()
        self.rows_host = self.rows_ring[turn]
        h = self.rows_host.numpy()
        h[0:M] = [self.cfg.real_token(int(t)) for t in tokens]
        h[R:R + M] = slots
        h[2 * R:2 * R + M] = pos
        run_start = np.zeros(M, dtype=np.int32)
        run_len = np.zeros(M, dtype=np.int32)
        i = 0
        while i < M:
            j = i
            while j + 1 < M and slots[j + 1] == slots[i] and pos[j + 1] == pos[j] + 1:
                j += 1
            run_start[i:j + 1] = i
            run_len[i] = j - i + 1
            i = j + 1
        h[3 * R:3 * R + M] = run_start
        h[4 * R:4 * R + M] = run_len
        if ctx3 is None:
            ctx3 = np.full((M, 3), -1, dtype=np.int32)
            ctx3[:, 0] = h[0:M]
        h[5 * R:5 * R + 3 * M] = np.asarray(ctx3, dtype=np.int32).reshape(-1)
        self.rows_dev.copy_(self.rows_host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.dev))
        self.rows_events[turn] = ev
        self.rows.M = M
        self.rows.max_groups = (int(max(pos)) + 1) // self.cfg.idx_ratio

    def launch(self, flags: int = 0, n_layers: int = -1):
        s = torch.cuda.current_stream(self.dev).cuda_stream
        rc = self.lib.qwrt_decode(C.byref(self.model), C.byref(self.rows), flags, n_layers, C.c_void_p(s))
        if rc != 0:
            raise RuntimeError(f"qwrt_decode failed: {rc}")

    def step(self, tokens, slots, pos, ctx3=None, flags: int = 0, graph: bool = False, n_layers: int = -1):
        """Run one batched step.  Returns nothing; results are in ``self.buf``."""
        self.stage_rows(tokens, slots, pos, ctx3)
        if self.guard_on and self.steps_run:
            self.check_guards()              # of the previous step (synchronises: a debugging mode)
        self.steps_run += 1
        if not graph:
            self.launch(flags, n_layers)
            return
        key = (len(tokens), flags, n_layers)
        g = self.graphs.get(key)
        if g is None:
            # score grid sized for the slot capacity so one graph serves every position
            self.rows.max_groups = self.model.d.ck_cap
            self.launch(flags, n_layers)            # warm-up outside capture (lazy module loading)
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.launch(flags, n_layers)
            self.graphs[key] = g
            # the warm-up executed the step once for real; the capture only records it
            return
        g.replay()

    # ---- guard zones (QW_GUARD): 64 KB of 0xA5 behind every step buffer, looked at after a step
    GUARD_BYTES = 64 * 1024

    def _zeros(self, name: str, shape, dtype) -> torch.Tensor:
        """A zeroed step buffer; with guard zones on, followed by a guard region that no kernel may touch
        (reference: src/engine/device_mem.hpp:26-58)."""
        if not self.guard_on:
            return torch.zeros(shape, dtype=dtype, device=self.dev)
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        pad = (-nbytes) % 256
        raw = torch.zeros(nbytes + pad + self.GUARD_BYTES, dtype=torch.uint8, device=self.dev)
        raw[nbytes:].fill_(0xA5)
        self.guards[name] = raw[nbytes:]
        self._guard_raw.append(raw)
        return raw[:nbytes].view(dtype).view(shape)

    def moe_balance(self, group=None, reset: bool = True):
        """Per layer: (pairs on the busiest rank, mean over ranks) since the last call - the imbalance expert parallelism
        pays at every layer (reference: src/engine/moe_balance.cpp:14-59).  None when the statistics are off."""
        if self.moe_stats is None:
            return None
        mine = self.moe_stats.clone()
        if reset:
            self.moe_stats.zero_()
        if self.sc.ranks > 1:
            import torch.distributed as dist
            allr = [torch.empty_like(mine) for _ in range(self.sc.ranks)]
            dist.all_gather(allr, mine, group=group)
            st = torch.stack(allr).float()
        else:
            st = mine.float()[None]
        return [(int(st[:, l].max()), float(st[:, l].mean())) for l in range(st.shape[1])]

    def check_guards(self) -> None:
        """Raise with the buffer's name if anything wrote behind a step buffer."""
        for name, g in self.guards.items():
            if not bool((g == 0xA5).all()):
                first = int((g != 0xA5).nonzero()[0])
                raise RuntimeError(f"guard zone behind buffer '{name}' was overwritten (first byte at +{first})")

    def check_error(self):
        """Raise if a kernel gave up on a bounded wait or failed a bounds check."""
        code, detail = self.err_word.tolist()
        if code:
            raise RuntimeError(f"device error word: code {code} detail {detail}")

    def set_comm(self, fn):
        """Install the collective hook (a Python callable wrapped as a C callback)."""
        self.comm_cb = S.COMM_FN(fn)
        self.model.comm = self.comm_cb
