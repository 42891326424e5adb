"""GPTQ calibration statistics: for every block (attention / MoE of every layer) the Hessian X^T X of its input rows,
accumulated in fp32 while prompts are prefilled, and written out for an offline quantiser
(reference: src/engine/calibrate.hip:18-66, which accumulates the same products with the library GEMM).

Offline tooling: the products run through torch.matmul."""
from __future__ import annotations

import os
from typing import Dict, Sequence, Tuple

import torch

from .engine import Engine


class Calibrator:
    def __init__(self, eng: Engine):
        if eng.dm.sc.ranks != 1 or eng.opts.prefill_chunk <= 0:
            raise ValueError("calibration runs on one GPU through the token-major prefill path")
        self.eng = eng
        self.H: Dict[Tuple[int, str], torch.Tensor] = {}
        self.rows: Dict[Tuple[int, str], int] = {}

    def _hook(self, layer: int, kind: str, x: torch.Tensor) -> None:
        xf = x.float()
        k = (layer, kind)
        if k not in self.H:
            self.H[k] = torch.zeros(xf.shape[1], xf.shape[1], dtype=torch.float32, device=xf.device)
            self.rows[k] = 0
        self.H[k].addmm_(xf.t(), xf)
        self.rows[k] += xf.shape[0]

    def run(self, slot: int, tokens: Sequence[int]) -> None:
        """Prefill ``tokens`` into ``slot`` (token-major path) and accumulate every block input's X^T X."""
        if len(tokens) < self.eng.opts.prefill_min:
            raise ValueError("prompt too short for the token-major path")
        from .prefill import Prefiller
        if self.eng.prefiller is None:
            self.eng.prefiller = Prefiller(self.eng.dm, chunk=min(self.eng.opts.prefill_chunk, max(256, self.eng.dm.slot_tokens)))
        self.eng.prefiller.on_block_input = self._hook
        try:
            self.eng.prefill(slot, tokens, want_logits=False)
        finally:
            self.eng.prefiller.on_block_input = None

    def dump(self, directory: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(directory, exist_ok=True)
        out = {f"layers.{l}.{kind}.hessian": h.cpu() for (l, kind), h in self.H.items()}
        out.update({f"layers.{l}.{kind}.rows": torch.tensor([n], dtype=torch.int64) for (l, kind), n in self.rows.items()})
        save_file(out, os.path.join(directory, "hessians.safetensors"))
