"""Engine runner: feed a prompt, print the greedy continuation, optionally write the per-position log-probability file in
the format of the CPU reference (`native/qw_ref --logprobs`), so the two can be diffed position by position
(reference: tools/qw_gpu.hip with --logprobs / --prefill-n / --token-by-token).

    python -m qwb200.tools.qw_gpu --model DIR [--ple DIR] --prompt 1,2,3 [--new 16] [--logprobs FILE] [--token-by-token]
                                  [--prefill-n N]      # the first N prompt tokens through the prefill path, the rest through decode steps:
                                                       # log-probabilities from position N - 1 on then test decoding on top of prefilled state
    python -m qwb200.tools.qw_gpu --synthetic tiny --prompt 5,6,7 --new 8"""
import argparse

import torch

from ..engine.engine import Engine, EngineOptions
from ..models.config import ModelConfig, check_hf_config


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--ple")
    ap.add_argument("--synthetic", choices=["tiny", "slice2", "full"])
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--new", type=int, default=0)
    ap.add_argument("--logprobs")
    ap.add_argument("--token-by-token", action="store_true", help="feed the prompt through decode steps instead of prefill")
    ap.add_argument("--weight-cache-dir")
    ap.add_argument("--prefill-n", type=int, default=0, help="prefill this many prompt tokens, feed the rest through decode steps")
    a = ap.parse_args()
    prompt = [int(t) for t in a.prompt.split(",")]
    opts = EngineOptions(slots=1, slot_tokens=max(1024, len(prompt) + a.new + 256), use_graphs=not a.token_by_token)
    if a.synthetic:
        cfg = {"tiny": ModelConfig.tiny, "slice2": ModelConfig.slice2, "full": ModelConfig.full}[a.synthetic]()
        eng = Engine.synthetic(cfg, opts, device="cuda:0", exact=(a.synthetic != "full"), ple_rows=1 << 16)
    else:
        from ..models.ple import PleTable
        cfg = ModelConfig.full()
        check_hf_config(cfg, a.model)
        table = PleTable.load(cfg, a.ple, pin=True) if a.ple else None
        eng = Engine.from_checkpoint(cfg, a.model, table, opts, weight_cache_dir=a.weight_cache_dir, log=print)
    lp = open(a.logprobs, "w") if a.logprobs else None
    toks = list(prompt)

    def record(pos, logits):
        if lp is None:
            return
        ls = torch.log_softmax(logits.float(), -1)
        top = int(ls.argmax())
        nxt = toks[pos + 1] if pos + 1 < len(toks) else top
        lp.write(f"{pos} {nxt} {float(ls[nxt]):.6f} {top} {float(ls[top]):.6f}\n")
    if 0 < a.prefill_n <= len(prompt) and not a.token_by_token:
        logits = eng.prefill(0, prompt[:a.prefill_n]).clone()
        record(a.prefill_n - 1, logits)
        for pos in range(a.prefill_n, len(prompt)):
            eng.decode([0], [prompt[pos]])
            logits = eng.dm.buf["logits"][0].clone()
            record(pos, logits)
    elif a.token_by_token or lp is not None:
        for pos, t in enumerate(prompt):              # every position's logits are wanted: one step per token
            eng.decode([0], [t])
            logits = eng.dm.buf["logits"][0].clone()
            record(pos, logits)
    else:
        logits = eng.prefill(0, prompt).clone()
    out = []
    for i in range(a.new):
        t = int(logits.argmax())
        out.append(t)
        toks.append(t)
        eng.decode([0], [t])
        logits = eng.dm.buf["logits"][0].clone()
        record(len(toks) - 1, logits)
    eng.dm.check_error()
    print(" ".join(map(str, out)))
    if lp:
        lp.close()


if __name__ == "__main__":
    main()
