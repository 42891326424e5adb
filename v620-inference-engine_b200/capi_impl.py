"""Python side of the C API shim (``native/src/capi.cpp``): one ``CApi`` object per ``qw_handle``.

Every method takes the C call's scalars and the *addresses* of its buffers, reads / writes them with
ctypes and forwards to the :class:`~qwb200.session.session.Session`.  ``open`` builds the engine from
the options JSON: ``model_dir`` (a checkpoint) or ``synthetic`` (``"full" | "slice2" | "tiny"``, random
weights), ``ple_dir`` or a synthetic table, ``slots`` (a list of capacities; the largest is used for all
slots), ``prefill_chunk``, ``host_cache_gb``, ``disk_cache_dir``, ``disk_cache_gb``, ``devices``, ``weight_cache_dir``, ``slot_spill``,
``warmup`` (capture every graph at start, default on), ``vision``.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import threading
from typing import List, Optional

import numpy as np


class QwSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float), ("repetition_penalty", C.c_float),
                ("seed", C.c_uint64)]


class QwCacheStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("hits", "tokens_restored", "snapshots_saved", "ram_bytes", "disk_bytes", "blocks",
                                          "snapshots", "prompt_tokens", "reused_tokens", "blend_candidate_tokens")]


class QwSlotTiming(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("restore_s", "prefill_s", "save_s", "pin_wait_s")]


class QwMedia(C.Structure):
    _fields_ = [("hash", C.c_uint64), ("video", C.c_int32), ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32),
                ("patches", C.POINTER(C.c_float)), ("starts", C.POINTER(C.c_int64))]


class QwStepReq(C.Structure):
    _fields_ = [("slot", C.c_int32), ("pending", C.c_int32), ("budget", C.c_int32), ("flags", C.c_int32), ("sampling", QwSampling)]


def _i32(addr: int, n: int) -> List[int]:
    if not addr or n <= 0:
        return []
    return np.ctypeslib.as_array(C.cast(addr, C.POINTER(C.c_int32)), shape=(n,)).tolist()


def _sampling(addr: int):
    from .engine.sampling import SamplingParams
    if not addr:
        return SamplingParams()
    s = QwSampling.from_address(addr)
    return SamplingParams(s.temperature, s.top_p, s.top_k, s.min_p, s.presence_penalty, s.frequency_penalty,
                          s.repetition_penalty, s.seed)


class SessionOps:
    """The calls of the C API on plain Python values, over one rank's Session.  With several GPUs every rank owns one of
    these and ``parallel.rank_group.RankGroup`` replays each call on all of them."""

    def __init__(self, session, vision=None):
        self.s, self.vision = session, vision

    def persist(self):
        self.s.persist()
        return 0

    def flush(self):
        self.s.store.flush()
        return 0

    def set_boundary_token(self, tok):
        self.s.set_boundary_token(tok)
        return 0

    def map_media(self, toks, media):
        """Every rank registers the prompt's media with its own vision front end (each runs the tower on the slices its
        prefill needs: same kernels on the same patches, so the ranks' embeddings are bit-identical) and maps the pad
        tokens to vision ids; the mapping is a pure function of the arguments, so all ranks return the same list."""
        return self.vision.map_media(toks, media) if self.vision is not None else list(toks)

    def acquire(self, toks, max_new):
        return self.s.acquire(toks, max_new)

    def release(self, slot):
        self.s.release(slot)
        return 0

    def begin_prompt(self, slot, toks):
        return self.s.begin_prompt(slot, toks)

    def prefetch(self, toks):
        return self.s.prefetch(toks)

    def prefill_some(self, slot, max_tokens):
        return bool(self.s.prefill_some(slot, max_tokens))

    def prefill_batch(self, slots, max_tokens):
        """One piece of every slot's prompt, one after the other (the chunked scan takes one sequence per chunk), in one
        call: on several ranks one round trip instead of one per slot."""
        return [bool(self.s.prefill_some(s_, m_)) for s_, m_ in zip(slots, max_tokens)]

    def sample_prompt(self, slot, sp):
        return self.s.sample_prompt(slot, sp)

    def decode(self, slots, tokens):
        self.s.decode(slots, tokens)
        return 0

    def sample_row(self, row, sp):
        return self.s.sample_row(row, sp)

    def set_stop_tokens(self, slot, ids):
        self.s.set_stop_tokens(slot, ids)
        return 0

    def generate(self, reqs, k):
        return self.s.generate(reqs, k)

    def check_error(self):
        self.s.e.dm.check_error()
        return 0


class CApi:
    def __init__(self, local: SessionOps, group=None):
        self.local = local              # rank 0's own session
        self.ops = group or local       # what engine calls go through: the rank group, or the local session alone
        self.group = group
        self.s = local.s
        self.vision = local.vision
        self._failure = ""
        self._lock = threading.Lock()

    # ---- lifetime / health
    def close(self):
        try:
            self.ops.flush()
        finally:
            if self.group is not None:
                self.group.shutdown()
            self.s = None

    def persist(self):
        return self.ops.persist()

    def failure(self) -> str:
        if self._failure:
            return self._failure
        if self.group is not None and self.group.failure():
            self._failure = self.group.failure()
            return self._failure
        try:
            self.s.e.dm.check_error()
        except RuntimeError as e:        # a kernel gave up on a bounded wait: sticky
            self._failure = str(e)
        return self._failure

    # ---- cache
    def set_boundary_token(self, tok):
        return self.ops.set_boundary_token(tok)

    def get_cache_stats(self, out):
        st = self.s.cache_stats()
        o = QwCacheStats.from_address(out)
        for n, _ in QwCacheStats._fields_:
            setattr(o, n, int(st.get(n, 0)))
        return 0

    def get_slot_timing(self, slot, out):
        t = self.s.slot_timing(slot)
        o = QwSlotTiming.from_address(out)
        for n, _ in QwSlotTiming._fields_:
            setattr(o, n, float(t.get(n, 0.0)))
        return 0

    # ---- slots / prompts
    def num_slots(self):
        return self.s.num_slots()

    def slot_capacity(self, slot):
        return self.s.slot_capacity(slot)

    def _tokens(self, addr, n, media_addr, n_media):
        toks = _i32(addr, n)
        if n_media and self.vision is not None:
            toks = self.ops.map_media(toks, self.vision.read_media(media_addr, n_media))
        return toks

    def acquire(self, addr, n, max_new, media, n_media):
        return self.ops.acquire(self._tokens(addr, n, media, n_media), max_new)

    def release(self, slot):
        return self.ops.release(slot)

    def begin_prompt(self, slot, addr, n, media, n_media):
        toks = self._tokens(addr, n, media, n_media)
        if n_media and self.vision is not None:
            self.vision.stage(slot, media, n_media)
        return self.ops.begin_prompt(slot, toks)

    def prefill_some(self, slot, max_tokens):
        return 1 if self.ops.prefill_some(slot, max_tokens) else 0

    def set_prompt(self, slot, addr, n, media, n_media):
        r = self.begin_prompt(slot, addr, n, media, n_media)
        while not self.ops.prefill_some(slot, 1 << 30):
            pass
        return r

    def prefetch(self, slot, addr, n, media, n_media):
        """Queue background disk reads for the prompt's stored prefix; returns the number of reads still pending."""
        self.ops.prefetch(self._tokens(addr, n, media, n_media))
        return self.s.loads_pending()

    def prefill_batch(self, n, slots, max_tokens, done):
        sl = _i32(slots, n)
        mt = np.ctypeslib.as_array(C.cast(max_tokens, C.POINTER(C.c_int64)), shape=(n,)).tolist()
        d = np.ctypeslib.as_array(C.cast(done, C.POINTER(C.c_int32)), shape=(n,))
        for i, ok in enumerate(self.ops.prefill_batch(sl, mt)):
            d[i] = 1 if ok else 0
        return 0

    def has_vision(self):
        return 1 if self.vision is not None else 0

    def has_mtp(self):
        return 1 if self.s.e.mtp else 0

    def sample_prompt(self, slot, p, lp):
        tok, l = self.ops.sample_prompt(slot, _sampling(p))
        if lp:
            C.c_float.from_address(lp).value = l
        return tok

    # ---- decoding
    def decode(self, n, slots, tokens):
        return self.ops.decode(_i32(slots, n), _i32(tokens, n))

    def sample_row(self, row, p, lp):
        tok, l = self.ops.sample_row(row, _sampling(p))
        if lp:
            C.c_float.from_address(lp).value = l
        return tok

    def set_stop_tokens(self, slot, ids, n):
        return self.ops.set_stop_tokens(slot, _i32(ids, n))

    def generate(self, n, reqs, k, tokens, logprobs, counts, first_rows, stopped):
        from .session.session import StepReq
        arr = (QwStepReq * n).from_address(reqs)
        rq = [StepReq(r.slot, r.pending, r.budget, r.flags, _sampling(C.addressof(r.sampling))) for r in arr]
        outs = self.ops.generate(rq, k)
        tk = np.ctypeslib.as_array(C.cast(tokens, C.POINTER(C.c_int32)), shape=(n * (k + 1),))
        lp = np.ctypeslib.as_array(C.cast(logprobs, C.POINTER(C.c_float)), shape=(n * (k + 1),))
        cn = np.ctypeslib.as_array(C.cast(counts, C.POINTER(C.c_int32)), shape=(n,))
        fr = np.ctypeslib.as_array(C.cast(first_rows, C.POINTER(C.c_int32)), shape=(n,))
        sp = np.ctypeslib.as_array(C.cast(stopped, C.POINTER(C.c_int32)), shape=(n,))
        for i, o in enumerate(outs):
            m = len(o.tokens)
            tk[i * (k + 1): i * (k + 1) + m] = o.tokens
            lp[i * (k + 1): i * (k + 1) + m] = o.logprobs
            cn[i], fr[i], sp[i] = m, o.first_row, int(o.stopped)
        return 0

    def _write_top(self, pair, k, ids, lps):
        i, l = pair
        m = min(k, len(i))
        np.ctypeslib.as_array(C.cast(ids, C.POINTER(C.c_int32)), shape=(k,))[:m] = i[:m]
        np.ctypeslib.as_array(C.cast(lps, C.POINTER(C.c_float)), shape=(k,))[:m] = l[:m]
        return m

    def top_logprobs(self, row, k, ids, lps):
        return self._write_top(self.s.top_logprobs(row, k), k, ids, lps)

    def top_logprobs_prompt(self, slot, k, ids, lps):
        return self._write_top(self.s.top_logprobs_prompt(slot, k), k, ids, lps)


def _free_port() -> int:
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def open(options_json: str) -> CApi:
    """Build engine + session from the options (see the module docstring).  ``devices`` with more than one entry
    starts one rank per device: rank 0 in this process, the others as worker processes that replay every call."""
    o = json.loads(options_json or "{}")
    devices = o.get("devices", [0])
    world = len(devices)
    if world == 1:
        return CApi(build_ops(o, 0, 1, 0))
    from .models.config import VALID_RANKS
    if world not in VALID_RANKS:
        raise ValueError(f"devices must list 1, 2, 4 or 8 GPUs, got {world}")
    from .parallel.rank_group import RankGroup
    port = _free_port()
    group = RankGroup.spawn(world, [], {"options": o, "master_port": port}, lambda: build_ops(o, 0, world, port),
                            ack_timeout=float(o.get("rank_timeout_s", 120)))
    return CApi(group.local, group)


def spill_plan(slots, slot_max_tokens: int, kv_spill: bool, dev_pages=None, host_pages: int = 0, page: int = 256, slot_spill=()):
    """(slot capacity in tokens, device pages or None, host pages) from the serving options.  Without spill every slot
    holds ``slot_max_tokens`` (or the largest entry of ``slots``) tokens in device memory.  With spill a slot's first
    max(slots) tokens stay in device memory and the rest live in pinned host pages; its capacity is ``slot_max_tokens``
    or, where ``slot_spill`` names tokens beyond a slot's device part (the reference's per-slot list; slots it does not
    name get ``slot_max_tokens - slots[i]``, src/engine/engine.hip:53-69), the largest ``slots[i] + slot_spill[i]``.
    The engine's slots are uniform: the reference's per-slot capacities become the largest of them.
    Explicit ``dev_pages`` / ``host_pages`` win."""
    n = len(slots)
    resident = max(int(x) for x in slots)
    cap = int(slot_max_tokens) if slot_max_tokens else resident
    if dev_pages is not None or host_pages:
        return cap, dev_pages, int(host_pages)
    spill = [int(x) for x in slot_spill]
    if len(spill) > n:
        raise ValueError("more slot_spill entries than slots")
    if spill:
        per = [int(slots[i]) + (spill[i] if i < len(spill) else max(0, int(slot_max_tokens) - int(slots[i]))) for i in range(n)]
        cap, kv_spill = max(per), True
    if not kv_spill or cap <= resident:
        return max(cap, resident) if not kv_spill else cap, None, 0
    cap_pages, res_pages = (cap + page - 1) // page, (resident + page - 1) // page
    return cap_pages * page, n * res_pages, n * (cap_pages - res_pages)


def build_ops(o: dict, rank: int, world: int, master_port: int) -> SessionOps:
    """One rank's engine + session from the options dictionary."""
    import torch
    from .engine.engine import Engine, EngineOptions
    from .models.config import ModelConfig
    from .session.session import Session
    o = dict(o)
    from .utils import settings as _settings
    st = _settings.Settings.from_env(prefill_chunk=o.get("prefill_chunk"), prefill_piece=o.get("prefill_piece"),
                                     host_cache_gb=o.get("host_cache_gb"), disk_cache_dir=o.get("disk_cache_dir"),
                                     disk_cache_gb=o.get("disk_cache_gb"), vision_cache_gb=o.get("vision_cache_gb"),
                                     weight_cache_dir=o.get("weight_cache_dir"), ple_dir=o.get("ple_dir"))
    _settings.set_current(st)
    import sys
    if rank == 0:
        print(st.describe(), file=sys.stderr, flush=True)
    if st.no_mtp:
        o["mtp"] = False
    if st.no_vision or world > 1:
        # the media descriptors can travel to the other ranks by value (SessionOps.map_media), but an image prompt on two
        # ranks has not run to completion yet: until it has, the vision tower serves one-rank engines
        o["vision"] = False
    o.setdefault("prefill_chunk", st.prefill_chunk)
    o.setdefault("prefill_piece", st.prefill_piece)
    if "host_cache_gb" not in o and "QW_HOST_CACHE_GB" in os.environ:
        o["host_cache_gb"] = st.host_cache_gb
    if st.disk_cache_dir and not o.get("disk_cache_dir"):
        o["disk_cache_dir"], o["disk_cache_gb"] = st.disk_cache_dir, st.disk_cache_gb
    slots = o.get("slots", [8192])
    if isinstance(slots, int):
        slots = [8192] * slots
    # KV spill: asked for by the option or QW_KV_SPILL, or implied by a per-slot list; QW_SPILL=0 forces it off
    slot_spill = (o.get("slot_spill") or st.slot_spill) if st.spill else []
    kv_spill = bool(o.get("kv_spill") or st.kv_spill or slot_spill) and st.spill
    cap, dev_pages, host_pages = spill_plan(slots, int(o.get("slot_max_tokens") or (st.slot_max_tokens if kv_spill else 0) or 0), kv_spill,
                                            o.get("dev_pages"), int(o.get("host_pages", 0)), slot_spill=slot_spill)
    devices = o.get("devices", [0])
    dev = f"cuda:{devices[rank]}"
    group = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(devices[rank])
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(master_port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        if not dist.is_initialized():
            # NCCL serves rendezvous and timing here, never the hot path: its in-switch (NVLS) transport is left off unless asked for,
            # so that a rank that dies does not leave its memory bound to a multicast object the other ranks still use
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=torch.device(dev))
    opts = EngineOptions(slots=len(slots), slot_tokens=cap, prefill_chunk=int(o.get("prefill_chunk", 4096)),
                         save_gdn=bool(o.get("mtp", True)), host_pages=host_pages, dev_pages=dev_pages, use_graphs=not st.nograph)
    log = (lambda m: print(m, file=sys.stderr, flush=True)) if rank == 0 else None
    def preflight(cfg):
        """Before anything slow: wait for a busy GPU if asked to, then refuse what cannot fit, with the numbers."""
        if not torch.cuda.is_available():
            return
        from .engine import memory_estimate as ME
        say = log or (lambda m: None)
        if st.start_wait_s > 0:
            ME.wait_for_device(lambda: torch.cuda.mem_get_info(devices[rank]), st.start_wait_s, say)
        if st.vram_check:
            plan = ME.estimate(cfg, world, slots=len(slots), slot_tokens=cap, dev_pages=dev_pages, host_pages=host_pages,
                               max_rows=opts.max_rows, prefill_chunk=opts.prefill_chunk, save_gdn=opts.save_gdn)
            say("memory estimate per GPU (GB): " + ", ".join(f"{k[:-3]} {v:.1f}" for k, v in plan.items()))
            ME.check(plan, torch.cuda.mem_get_info(devices[rank])[1], ME.host_available_bytes(), local_ranks=world)
    if "model_dir" in o and o["model_dir"]:
        from .models.config import check_hf_config
        from .models.ple import PleTable
        cfg = ModelConfig.full()
        check_hf_config(cfg, o["model_dir"])
        preflight(cfg)
        table = PleTable.load(cfg, o["ple_dir"], pin=st.ple_pin) if o.get("ple_dir") else None
        eng = Engine.from_checkpoint(cfg, o["model_dir"], table, opts, ranks=world, rank=rank, device=dev,
                                     weight_cache_dir=o.get("weight_cache_dir") or st.weight_cache_dir or None, log=log)
    else:
        kind = o.get("synthetic", "tiny")
        cfg = {"full": ModelConfig.full, "slice2": ModelConfig.slice2, "tiny": ModelConfig.tiny}[kind]()
        preflight(cfg)
        eng = Engine.synthetic(cfg, opts, ranks=world, rank=rank, device=dev, exact=(kind != "full"),
                               ple_rows=int(o.get("ple_rows", 1 << 16)), ple_pinned=torch.cuda.is_available())
    if world > 1:
        from .parallel.dist_engine import attach_p2p, attach_tp, set_fused
        attach_p2p(eng)
        set_fused(True)
        attach_tp(eng)
    if o.get("warmup", True) and torch.cuda.is_available():
        n_graphs = eng.warmup(max_rows=int(o.get("warmup_rows", 8)))
        if rank == 0:
            print(f"engine: {n_graphs} graphs captured; memory plan {eng.memory_plan()}", file=sys.stderr, flush=True)
    disk = o.get("disk_cache_dir") or None
    if disk and world > 1:
        disk = os.path.join(disk, f"rank{rank}")          # every rank keeps the blocks of its own shard
        os.makedirs(disk, exist_ok=True)
    ses = Session(eng, host_cache_bytes=int(float(o.get("host_cache_gb", 8)) * (1 << 30)),
                  disk_cache_dir=disk,
                  disk_cache_bytes=int(float(o.get("disk_cache_gb", 0)) * (1 << 30)),
                  prefill_piece=int(o.get("prefill_piece", 2048)))
    vision = None
    if o.get("vision", True) and torch.cuda.is_available():
        from .vision import VisionConfig, VisionEncoder, VisionFrontend, synth_vision_weights
        enc = None
        if o.get("model_dir"):
            enc = VisionEncoder.from_checkpoint(o["model_dir"], dev)
        elif o.get("vision") == "synthetic":
            vc = VisionConfig(depth=int(o.get("vision_depth", 2)), out_dim=cfg.hidden)
            enc = VisionEncoder(vc, synth_vision_weights(vc, seed=1), dev)
        if enc is not None:
            vision = VisionFrontend(enc, int(float(o.get("vision_cache_gb", st.vision_cache_gb)) * (1 << 30)))
            eng.vision_lookup = vision.lookup
    return SessionOps(ses, vision)
