"""KV spill: a slot whose later pages live in pinned host memory decodes exactly like a fully resident one
(the reference checks the same in tests/gpu/test_spill.hip: bit-exact resident vs spilled)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_spilled_slot_equals_resident_slot():
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    cfg = ModelConfig.tiny()
    toks = [(i * 13 + 7) % 900 + 5 for i in range(700)]          # three KV pages of 256 tokens
    outs = []
    for opts in (EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=0),
                 EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=0, dev_pages=1, host_pages=3)):
        eng = Engine.synthetic(cfg, opts, device="cuda:0", exact=True, ple_rows=4096, seed=3)
        lg = eng.prefill(0, toks).clone()
        t = int(lg.argmax())
        seq = []
        for _ in range(8):
            t = eng.decode([0], [t])[0]
            seq.append(t)
        torch.cuda.synchronize()
        eng.dm.check_error()
        outs.append((lg, seq, eng))
    spilled = outs[1][2].dm
    assert spilled.n_host_pages == 3 and spilled.n_dev_pages == 1
    assert int((spilled.page_table_host[0, :3] >= spilled.n_dev_pages).sum()) >= 2      # pages 1 and 2 of the slot sit in host memory
    assert torch.equal(outs[0][0], outs[1][0])
    assert outs[0][1] == outs[1][1]
