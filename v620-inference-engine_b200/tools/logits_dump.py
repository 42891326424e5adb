"""Bit-exact build-to-build check: dump the logits of a fixed run, compare two dumps.

``dump`` prefills a fixed random prompt, decodes ``--new`` greedy tokens and writes, per position, the sha256 of the
fp32 logits row, its argmax and its log-sum-exp, plus the raw rows of the first and last position.  Two builds that
claim to compute the same thing (a refactor, a scheduling change, a different launch configuration) must produce
identical files; ``compare`` prints the first position where they do not and how far apart the kept rows are.
(Role of the reference's bench/logits_dump.hip and the diff step of bench/run_suite.sh.)

    python -m qwb200.tools.logits_dump dump out.json --synthetic slice2 --prompt-len 256 --new 32
    python -m qwb200.tools.logits_dump compare a.json b.json
"""
from __future__ import annotations

import argparse
import hashlib
import json
from typing import List


def row_record(logits) -> dict:
    import torch
    x = logits.detach().float().cpu().contiguous()
    return {"sha256": hashlib.sha256(x.numpy().tobytes()).hexdigest(), "argmax": int(x.argmax()),
            "lse": float(torch.logsumexp(x, -1))}


def compare(a: dict, b: dict) -> dict:
    """``{"identical", "positions", "first_diff", "argmax_diffs", "kept_max_abs"}`` for two dumps of the same run."""
    if a["run"] != b["run"]:
        return {"identical": False, "error": f"different runs: {a['run']} vs {b['run']}"}
    ra, rb = a["rows"], b["rows"]
    n = min(len(ra), len(rb))
    diff = [i for i in range(n) if ra[i]["sha256"] != rb[i]["sha256"]]
    kept = 0.0
    for k in ("first_row", "last_row"):
        if k in a and k in b and len(a[k]) == len(b[k]):
            kept = max(kept, max((abs(x - y) for x, y in zip(a[k], b[k])), default=0.0))
    return {"identical": not diff and len(ra) == len(rb), "positions": n, "first_diff": diff[0] if diff else None,
            "n_diff": len(diff), "argmax_diffs": sum(ra[i]["argmax"] != rb[i]["argmax"] for i in range(n)), "kept_max_abs": kept}


def dump(a) -> dict:
    import torch
    from ..engine.engine import Engine, EngineOptions
    from ..models.config import ModelConfig
    cfg = {"tiny": ModelConfig.tiny, "slice2": ModelConfig.slice2, "full": ModelConfig.full}[a.synthetic]()
    opts = EngineOptions(slots=1, slot_tokens=max(1024, a.prompt_len + a.new + 64), use_graphs=not a.no_graphs)
    eng = Engine.synthetic(cfg, opts, device="cuda:0", exact=(a.synthetic != "full"), ple_rows=1 << 16, seed=a.seed)
    g = torch.Generator().manual_seed(a.seed)
    prompt = torch.randint(0, min(cfg.vocab, 200000), (a.prompt_len,), generator=g).tolist()
    rows: List[dict] = []
    logits = eng.prefill(0, prompt).clone()
    first = logits.float().cpu().tolist()
    rows.append(row_record(logits))
    for _ in range(a.new):
        eng.decode([0], [rows[-1]["argmax"]])
        logits = eng.dm.buf["logits"][0].clone()
        rows.append(row_record(logits))
    eng.dm.check_error()
    return {"run": {"model": a.synthetic, "prompt_len": a.prompt_len, "new": a.new, "seed": a.seed, "graphs": not a.no_graphs},
            "rows": rows, "first_row": first, "last_row": logits.float().cpu().tolist()}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("dump")
    d.add_argument("out")
    d.add_argument("--synthetic", choices=["tiny", "slice2", "full"], default="slice2")
    d.add_argument("--prompt-len", type=int, default=256)
    d.add_argument("--new", type=int, default=32)
    d.add_argument("--seed", type=int, default=0)
    d.add_argument("--no-graphs", action="store_true")
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    a = ap.parse_args(argv)
    if a.cmd == "dump":
        out = dump(a)
        with open(a.out, "w") as f:
            json.dump(out, f)
        print(f"{len(out['rows'])} positions -> {a.out}; last argmax {out['rows'][-1]['argmax']}")
        return 0
    with open(a.a) as f:
        da = json.load(f)
    with open(a.b) as f:
        db = json.load(f)
    r = compare(da, db)
    print(json.dumps(r))
    return 0 if r["identical"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
