"""Where do token-major prefill and step-wise decode drift apart?  Divergence of the two paths by depth.

Both paths compute the same function with different kernels (tcgen05 GEMMs over all tokens against per-token GEMVs, a
sequential scan against a single state update, ...), so their logits differ by rounding.  When a change makes them
differ by more than that, this tool says in which layer it starts: for depth n = 1 .. n_layers the model is cut after
n layers (the final mixer and the output head applied to the cut stack), the prompt's last token is evaluated once by
the prefill path (slot 0, whole prompt) and once by the decode path (slot 1, the prompt fed token by token, recurrent
state restored before every probe), and the two logit rows are compared.  A layer's state depends only on the layers
below it, so the cut does not disturb the layers that are kept.
(Role of the reference's tools/qw_layer_diff.hip.)

    python -m qwb200.tools.layer_diff --synthetic tiny --prompt-len 96
    python -m qwb200.tools.layer_diff --model DIR --ple DIR --prompt 1,2,3,... --depths 1,2,4,8,16,32,48
"""
from __future__ import annotations

import argparse
from typing import List, Optional, Sequence

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine.state_io import StateIO
from ..models.config import ModelConfig, check_hf_config


def depth_divergence(eng: Engine, prompt: Sequence[int], depths: Optional[Sequence[int]] = None) -> List[dict]:
    """Rows ``{depth, layer_kind, max_abs, rel, kl, same_top}``: prefill-vs-decode difference of the last token's logits
    with the stack cut after ``depth`` layers.  ``eng`` needs two slots, one rank, token-major prefill on, no graphs."""
    from ..engine.prefill import Prefiller
    cfg = eng.cfg
    if eng.dm.sc.ranks != 1 or eng.opts.slots < 2 or eng.opts.prefill_chunk <= 0:
        raise ValueError("layer_diff wants one rank, two slots and the token-major prefill path")
    if len(prompt) < max(2, eng.opts.prefill_min):
        raise ValueError("prompt shorter than the token-major path's minimum")
    depths = list(depths) if depths else list(range(1, cfg.n_layers + 1))
    if eng.prefiller is None:
        eng.prefiller = Prefiller(eng.dm, chunk=min(eng.opts.prefill_chunk, max(256, eng.dm.slot_tokens)))
    io = StateIO(eng.dm)
    # decode side: everything but the last token at full depth, then keep the recurrent state
    eng.reset(1)
    for t in prompt[:-1]:
        eng.decode([1], [int(t)])
    snap = io.snapshot_save(1)
    pos = len(prompt) - 1
    ctx3 = eng._ctx3(1, [prompt[-1]])
    rows = []
    for n in depths:
        io.snapshot_restore(1, snap)
        eng.dm.step([int(prompt[-1])], [1], [pos], ctx3, graph=False, n_layers=n)
        dec = eng.dm.buf["logits"][0].float().clone()
        eng.reset(0)
        eng.prefiller.layer_limit = n
        try:
            pre = eng.prefill(0, list(prompt)).float().clone()
        finally:
            eng.prefiller.layer_limit = None
        eng.dm.check_error()
        lp, ld = torch.log_softmax(pre, -1), torch.log_softmax(dec, -1)
        rows.append({"depth": n, "layer_kind": "qsa" if cfg.is_qsa(n - 1) else "gdn",
                     "max_abs": float((pre - dec).abs().max()), "rel": float((pre - dec).norm() / dec.norm().clamp_min(1e-30)),
                     "kl": float((ld.exp() * (ld - lp)).sum()), "same_top": bool(int(pre.argmax()) == int(dec.argmax()))})
    io.snapshot_restore(1, snap)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model")
    ap.add_argument("--ple")
    ap.add_argument("--synthetic", choices=["tiny", "slice2", "full"])
    ap.add_argument("--prompt", help="comma-separated token ids")
    ap.add_argument("--prompt-len", type=int, default=96, help="random prompt of this length when --prompt is absent")
    ap.add_argument("--depths", help="comma-separated depths (default: every layer)")
    ap.add_argument("--weight-cache-dir")
    a = ap.parse_args(argv)
    opts = EngineOptions(slots=2, slot_tokens=1024, use_graphs=False)
    if a.synthetic:
        cfg = {"tiny": ModelConfig.tiny, "slice2": ModelConfig.slice2, "full": ModelConfig.full}[a.synthetic]()
        eng = Engine.synthetic(cfg, opts, device="cuda:0", exact=(a.synthetic != "full"), ple_rows=1 << 16)
    else:
        from ..models.ple import PleTable
        cfg = ModelConfig.full()
        check_hf_config(cfg, a.model)
        table = PleTable.load(cfg, a.ple, pin=True) if a.ple else None
        eng = Engine.from_checkpoint(cfg, a.model, table, opts, weight_cache_dir=a.weight_cache_dir, log=print)
    if a.prompt:
        prompt = [int(t) for t in a.prompt.split(",")]
    else:
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, min(cfg.vocab, 200000), (a.prompt_len,), generator=g).tolist()
    depths = [int(d) for d in a.depths.split(",")] if a.depths else None
    print("depth kind   max|dlogit|   rel.err      KL(dec||pre)  same argmax")
    for r in depth_divergence(eng, prompt, depths):
        print(f"{r['depth']:5d} {r['layer_kind']:4s} {r['max_abs']:12.5f} {r['rel']:11.3e} {r['kl']:13.3e}  {r['same_top']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
