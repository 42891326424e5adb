"""The C++ fp32 reference (native/src/ref_model.hpp, native/qw_ref) against the PyTorch oracle on a small random
checkpoint written in the checkpoint's own format: per-expert tensors, the language-model prefix, config.json and a
PLE table directory."""
import dataclasses
import json
import os
import subprocess

import numpy as np
import torch


def write_checkpoint(cfg, w, table, d):
    from safetensors.torch import save_file
    from qwb200.models.weights import PREFIX
    out = {}
    for n, t in w.items():
        if n.startswith("mtp."):
            continue
        if ".mlp.experts." in n:
            head, tail = n.split(".mlp.experts.")
            for e in range(t.shape[0]):
                out[f"{PREFIX}{head}.mlp.experts.{e}.{tail}"] = t[e].contiguous()
        else:
            out[PREFIX + n] = t.contiguous()
    os.makedirs(d, exist_ok=True)
    save_file(out, os.path.join(d, "model-00001-of-00001.safetensors"))
    q = {k: v for k, v in dataclasses.asdict(cfg).items() if isinstance(v, (int, float)) and not isinstance(v, bool)}
    q["ngram_vocab_base"], q["ple_seed"] = cfg.ngram_vocab_base, cfg.ple_seed
    if cfg.layer_types:
        q["layer_types"] = list(cfg.layer_types)
    json.dump({"qw": q}, open(os.path.join(d, "config.json"), "w"))
    table.save(os.path.join(d, "ple"))


def test_cpp_reference_matches_pytorch_oracle(tmp_path):
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.reference import RefModel
    from qwb200.models.weights import synth_weights
    from qwb200.native import build as nb
    nb.build()
    cfg = ModelConfig.tiny(idx_budget=16)          # a 40-token prompt passes the budget: the indexer's selection runs
    w = synth_weights(cfg, seed=5)
    table = PleTable.synthetic(cfg, rows=2048, layout="bf16", seed=5)
    d = str(tmp_path / "ckpt")
    write_checkpoint(cfg, w, table, d)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(9)).tolist()
    ref = RefModel(cfg, w, table)
    st = ref.new_state()
    want = ref.forward(st, prompt)[0].numpy()
    nxt = int(want.argmax())
    dump, lp = str(tmp_path / "logits.bin"), str(tmp_path / "lp.txt")
    r = subprocess.run([nb.REF_EXE, "--model", d, "--ple", os.path.join(d, "ple"), "--prompt", ",".join(map(str, prompt)), "--new", "1",
                        "--logprobs", lp, "--dump-logits", dump, "--threads", "4"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert int(r.stdout.split()[0]) == nxt                      # greedy token after the prompt
    lines = [l.split() for l in open(lp).read().strip().splitlines()]
    assert len(lines) == 41 and [int(l[0]) for l in lines] == list(range(41))
    assert [int(l[1]) for l in lines[:39]] == prompt[1:]
    row = lines[39]                                             # the last prompt position predicts the greedy token
    lsm = torch.log_softmax(torch.from_numpy(want), -1)
    assert int(row[1]) == nxt and int(row[3]) == nxt and abs(float(row[2]) - float(lsm[nxt])) < 2e-3
    # raw logits of the last fed position (the generated token) against the oracle fed the same token
    want2 = ref.forward(st, [nxt])[0].numpy()
    got2 = np.fromfile(dump, dtype=np.float32)
    assert got2.shape == want2.shape
    assert np.abs(got2 - want2).max() / np.abs(want2).max() < 2e-3
