"""The bounds-checked build of the kernels (``libqw_kernels_checked.so``, selected with QW_DEVICE_CHECKS=1): a tiny
model decodes exactly as with the plain build, and an index that is out of range by construction of the test - a token id
beyond the vocabulary, a position beyond the slot's page table - is reported through the error word with the kernel
skipping the access (nothing is read or written out of bounds, nothing traps)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes as C, sys
import torch
import qwb200
from qwb200.engine.engine import Engine, EngineOptions
from qwb200.models.config import ModelConfig
from qwb200.ops import lib as qlib
L = qlib.load(True)
L.qwk_device_checks.restype = C.c_int
checked = int(L.qwk_device_checks())
cfg = ModelConfig.tiny()
eng = Engine.synthetic(cfg, EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=128), exact=True, ple_rows=2048)
prompt = [(i * 7 + 3) % 900 + 5 for i in range(150)]
eng.prefill(0, prompt)
tok = int(eng.dm.buf["amax_idx"][0])
out = []
for _ in range(8):
    tok = eng.decode([0], [tok])[0]
    out.append(tok)
eng.dm.check_error()
print("TOKENS", checked, out)
if checked:
    dm, s = eng.dm, C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())
    # a token id beyond the vocabulary: reported, the row is left as it was
    X = torch.full((2, cfg.hc, cfg.hidden), 7.0, device=dm.dev)
    toks = torch.tensor([5, cfg.vocab + 9], dtype=torch.int32, device=dm.dev)
    assert L.qwk_embed_rows(P(toks), P(dm.globals_w["embed"]), cfg.hidden, 0, cfg.hidden, cfg.hc, cfg.vocab, P(X), 2, s) == 0
    torch.cuda.synchronize()
    code, detail = dm.err_word.tolist()
    assert code == 2 and (detail & 0xffffffff) == (0x01000000 | 1), (code, hex(detail & 0xffffffff))
    assert bool((X[1] == 7.0).all()) and not bool((X[0] == 7.0).all())
    dm.err_word.zero_()
    # a position beyond the slot's pages: the prep kernel reports and writes no key / value row
    d, sc = dm.model.d, dm.sc
    rows = torch.zeros(8, dtype=torch.int32, device=dm.dev)       # slot 0 | pos | run_start | run_len
    bad = d.max_pages * 256 + 3
    rows[1] = bad
    rows[3] = 1
    k_before = dm.k_dev[0].clone()
    lw = dm.layers_w[cfg.qsa_layers[0]]
    proj = torch.randn(1, sc.qsa_proj_l, device=dm.dev)
    rc = L.qwk_qsa_prep(P(proj), sc.qsa_proj_l, sc.qh_l, sc.kvh_l, cfg.idx_heads, P(lw["qn1"]), P(lw["kn1"]), P(lw["iqn1"]), P(lw["ikn1"]), 1,
                        P(rows[0:1]), P(rows[1:2]), P(rows[2:3]), P(rows[3:4]), P(dm.k_dev[0]), P(dm.v_dev[0]), None, None, d.n_dev_pages,
                        P(dm.page_table), d.max_pages, P(dm.buf["q"]), P(dm.buf["iq"]), P(dm.raw_ring[0]), P(dm.ck[0]), d.ck_cap,
                        cfg.idx_ratio, C.c_float(cfg.eps), s)
    assert rc == 0
    torch.cuda.synchronize()
    code, detail = dm.err_word.tolist()
    assert code == 2 and ((detail & 0xffffffff) >> 24) == 2, (code, hex(detail & 0xffffffff))
    assert torch.equal(dm.k_dev[0], k_before)
    dm.err_word.zero_()
    tok2 = eng.decode([0], [tok])[0]            # the engine carries on
    eng.dm.check_error()
    print("CHECKS OK")
'''


def run_child(checked: bool):
    env = dict(os.environ, PYTHONPATH=ROOT, QW_DEVICE_CHECKS="1" if checked else "0")
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.gpu
def test_checked_build_decodes_like_the_plain_one_and_reports_bad_indices():
    plain = run_child(False)
    chk = run_child(True)
    line = lambda out: [l for l in out.splitlines() if l.startswith("TOKENS")][0].split(" ", 2)
    assert line(plain)[1] == "0" and line(chk)[1] == "1"
    assert line(plain)[2] == line(chk)[2]
    assert "CHECKS OK" in chk
