"""How often does a decode step select a spilled group that a recent step selected too?

    python -m qwb200.tools.spill_locality [--tokens 65536] [--resident 16384] [--steps 256] [--layers 0]

Fills one slot with ``--tokens`` tokens of which ``--resident`` live in device memory, decodes ``--steps`` tokens one
row at a time and reads back, after every step, the groups the last sparse-attention layer selected.  Prints the share
of selected groups that lie in host memory and, of those, the share selected again within 1, 2, 4, ..., 32 positions:
the hit rate a cache of recently fetched groups can reach, which is what decided for the device cache in front of
the spilled pages (``spill_cache_mb``).  With random weights and tokens the selection is close to uniform, so the
figures are a floor; real text re-selects far more.
(The reference's experiment: QW_SPILL_LOCALITY counters, src/kernels/qsa.hip:293-339.)"""
import argparse
import dataclasses
import json

import torch

from ..engine.engine import Engine, EngineOptions
from ..engine import device_model as DM
from ..models.config import ModelConfig
from ..utils.locality import LocalityCounter, spilled_groups


def selected_groups(dm, row: int, pos: int):
    """Groups the last QSA layer selected for decode row ``row`` at position ``pos`` (a dense step selects them all)."""
    n = int(dm.buf["sel_n"][row].item())
    if n < 0:
        return range((pos + 1) // dm.cfg.idx_ratio)
    return dm.buf["sel"][row, :n].cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--resident", type=int, default=16384)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0)
    a = ap.parse_args()
    cfg = ModelConfig.full()
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    page = DM.KV_PAGE
    cap = (a.tokens + a.steps + 2 * page - 1) // page * page
    res_pages, max_pages = a.resident // page, cap // page
    eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=cap, use_graphs=False, prefill_chunk=4096, dev_pages=res_pages,
                                              host_pages=max_pages - res_pages), device="cuda:0", ple_rows=1 << 20)
    g = torch.Generator().manual_seed(9)
    eng.prefill(0, torch.randint(0, cfg.vocab, (a.tokens,), generator=g).tolist(), want_logits=True)
    spilled = spilled_groups(eng.dm.page_table_host[0].numpy(), eng.dm.n_dev_pages, page, cfg.idx_ratio)
    cnt = LocalityCounter(len(spilled))
    tok = 11
    for i in range(a.steps):
        pos = a.tokens + i
        tok = eng.decode([0], [tok])[0]
        torch.cuda.synchronize()
        cnt.step(pos, selected_groups(eng.dm, 0, pos), spilled)
    eng.dm.check_error()
    out = {"tokens": a.tokens, "resident": a.resident, "layers": cfg.n_layers, **cnt.report()}
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
