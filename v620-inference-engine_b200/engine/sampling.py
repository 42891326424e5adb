"""Sampling front end: the GPU sampler kernel for every row, the native host sampler for rows the
kernel hands back (nucleus wider than its 256 candidates) — the contract of the reference's
``sample_candidates`` / ``sample_token`` pair (src/session/sampling.cpp:142-261, generate.cpp:213-249)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..native import host as H


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0

    def has_penalties(self) -> bool:
        return self.presence_penalty != 0 or self.frequency_penalty != 0 or self.repetition_penalty != 1

    def to_host(self) -> H.Sampling:
        return H.Sampling.make(self.temperature, self.top_p, self.top_k, self.min_p, self.presence_penalty,
                               self.frequency_penalty, self.repetition_penalty, self.seed)


_PARAM_DT = np.dtype([("temperature", "f4"), ("top_p", "f4"), ("top_k", "i4"), ("min_p", "f4"), ("presence", "f4"),
                      ("frequency", "f4"), ("repetition", "f4"), ("_pad", "i4"), ("seed", "u8"), ("slot", "i4"),
                      ("position", "i4")])
_OUT_DT = np.dtype([("token", "i4"), ("logprob", "f4"), ("fallback", "i4"), ("lse", "f4")])
assert _PARAM_DT.itemsize == 48 and _OUT_DT.itemsize == 16


class GpuSampler:
    def __init__(self, lib, device, vocab: int, slots: int, max_rows: int, seed: int = 0):
        self.lib, self.dev, self.V, self.slots = lib, torch.device(device), vocab, slots
        self.gen = torch.zeros((slots, vocab), dtype=torch.int16, device=self.dev)
        self.seen = torch.zeros((slots, vocab), dtype=torch.uint8, device=self.dev)
        self.params_host = torch.zeros(max_rows * 48, dtype=torch.uint8).pin_memory()
        self.params_dev = torch.zeros(max_rows * 48, dtype=torch.uint8, device=self.dev)
        self.out_dev = torch.zeros(max_rows * 16, dtype=torch.uint8, device=self.dev)
        self.out_host = torch.zeros(max_rows * 16, dtype=torch.uint8).pin_memory()
        self.host = H.HostSampler(seed)
        self.rng = np.random.default_rng(seed)
        self.fallbacks = 0
        self.host_only = False          # QW_GPU_SAMPLING=0: every row is drawn by the host sampler (a diagnostic: one logits row copied per draw)

    def reset_slot(self, slot: int):
        self.gen[slot].zero_()
        self.seen[slot].zero_()

    def note_tokens(self, slot: int, tokens: Sequence[int], generated: bool):
        """The tokens join the slot's sequence (prompt tokens only count for the repetition penalty)."""
        if not len(tokens):
            return
        t = torch.as_tensor([x for x in tokens if 0 <= x < self.V], dtype=torch.long, device=self.dev)
        self.seen[slot].index_fill_(0, t, 1)
        if generated:
            self.gen[slot].index_add_(0, t, torch.ones_like(t, dtype=torch.int16))

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], slots: Sequence[int], positions: Sequence[int],
               hists: Optional[Sequence[Tuple[Sequence[int], int]]] = None,
               force_host: Optional[Sequence[bool]] = None) -> Tuple[List[int], List[float]]:
        """logits fp32 [M, V] on the device.  ``hists[i] = (tokens so far, prompt_end)`` is only needed for a host fallback;
        ``force_host[i]``: draw row i on the host from ``hists[i]`` (rows whose penalty counts must include tokens that
        are not in the slot's count tables yet)."""
        M = len(params)
        arr = np.zeros(M, dtype=_PARAM_DT)
        for i, (p, s, pos) in enumerate(zip(params, slots, positions)):
            seed = p.seed if p.seed else int(self.rng.integers(1, 2**63 - 1))
            arr[i] = (p.temperature, p.top_p, p.top_k, p.min_p, p.presence_penalty, p.frequency_penalty,
                      p.repetition_penalty, 0, seed, s if p.has_penalties() else -1, pos)
        self.params_host[:M * 48].copy_(torch.from_numpy(arr.view(np.uint8)))
        self.params_dev[:M * 48].copy_(self.params_host[:M * 48], non_blocking=True)
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        rc = self.lib.qwk_sample(C.c_void_p(logits.data_ptr()), logits.stride(0), logits.shape[1], M,
                                 C.c_void_p(self.params_dev.data_ptr()), C.c_void_p(self.gen.data_ptr()),
                                 C.c_void_p(self.seen.data_ptr()), C.c_void_p(self.out_dev.data_ptr()), st)
        if rc != 0:
            raise RuntimeError(f"qwk_sample failed: {rc}")
        self.out_host[:M * 16].copy_(self.out_dev[:M * 16], non_blocking=True)
        torch.cuda.current_stream(self.dev).synchronize()
        out = self.out_host[:M * 16].numpy().view(_OUT_DT)
        toks, lps = [int(x) for x in out["token"]], [float(x) for x in out["logprob"]]
        for i in range(M):
            if out["fallback"][i] or self.host_only or (force_host is not None and force_host[i]):
                self.fallbacks += 1
                hist, pend = hists[i] if hists else ((), 0)
                toks[i], lps[i] = self.host.sample(logits[i].float().cpu().numpy(), params[i].to_host(), hist, pend)
        return toks, lps
