"""Several tensor-parallel ranks emulated in one process on one GPU, for tests of the multi-rank token-major prefill.

Every emulated rank is a complete ``Engine`` of its shard (own weights slice, own slot state, own prefill buffers);
their prefill channels are plain tensors of this process that name one another as peers.  A chunk's jobs are handed
to ``qwrt_prefill`` together, which issues each kernel for all ranks before the next one on one stream: a kernel that
waits for other ranks' data always finds it complete, so nothing ever spins on a GPU that runs one kernel at a time.
What this exercises is everything but the NVLink transport: the sharded kernels, the collectives' addressing,
sequencing and rank-order sums, and the runtime's schedule.  Decode steps of a multi-rank engine are one native call
per rank that waits for its peers inside, so they are not emulated here (they run as one process per GPU).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine.prefill import Prefiller
from ..models.config import ModelConfig
from . import tp_channel


class EmulatedRanks:
    def __init__(self, cfg: ModelConfig, weights, table, opts: EngineOptions, ranks: int, device: str = "cuda:0"):
        self.ranks = ranks
        self.engines: List[Engine] = [Engine.from_weights(cfg, weights, table, opts, ranks=ranks, rank=r, device=device)
                                      for r in range(ranks)]
        rows = min(opts.prefill_chunk, max(256, self.engines[0].dm.slot_tokens))
        chans = tp_channel.make_emulated(cfg, ranks, rows, torch.device(device), bool(cfg.mtp) and self.engines[0].mtp)
        for e, ch in zip(self.engines, chans):
            e.tp_channels = [ch]
            # the library reports to the error word registered last: every emulated rank looks at that one
            e.dm.err_word = self.engines[-1].dm.err_word

    def prefill(self, slot: int, tokens: Sequence[int], want_logits: bool = True) -> Optional[int]:
        """Append ``tokens`` to ``slot`` on every rank; returns the greedy next token (merged over the vocabulary shards)."""
        toks = [int(t) for t in tokens]
        gens = [e.prefill_jobs(slot, toks, want_logits) for e in self.engines]
        lib = self.engines[0].dm.lib
        while True:
            jobs = []
            for g in gens:
                try:
                    jobs.append(next(g))
                except StopIteration:
                    pass
            if not jobs:
                break
            if len(jobs) != self.ranks:
                raise RuntimeError("emulated ranks fell out of step")
            Prefiller.launch(lib, jobs)
        torch.cuda.synchronize()
        for e in self.engines:
            e.dm.check_error()
        return int(self.engines[0].dm.buf["amax_idx"][0]) if want_logits else None

    def logits(self) -> torch.Tensor:
        """The last prefill's logits over the whole vocabulary (the ranks' shards side by side)."""
        return torch.cat([e.dm.buf["logits"][0] for e in self.engines])
