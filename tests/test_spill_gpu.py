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


def _run(opts, toks, n_new, seed=3):
    from qwb200.engine.engine import Engine
    from qwb200.models.config import ModelConfig
    eng = Engine.synthetic(ModelConfig.tiny(), opts, device="cuda:0", exact=True, ple_rows=4096, seed=seed)
    out = []
    for prompt in toks:                              # several prompts one after the other in slot 0: the slot is reused
        eng.reset(0)
        lg = eng.prefill(0, prompt).clone()
        t = int(lg.argmax())
        seq = [t]
        for _ in range(n_new):
            t = eng.decode([0], [t])[0]
            seq.append(t)
        out.append((lg, seq))
    torch.cuda.synchronize()
    eng.dm.check_error()
    return eng, out


@pytest.mark.parametrize("cache_mb,graphs", [(256, False), (256, True), (0, False)])
def test_spill_cache_hits_and_stays_exact(cache_mb, graphs):
    """The device cache in front of the host pages serves repeated reads (hits counted), leaves the results bit-exact,
    and a slot that is filled again with other tokens does not see rows of the earlier request."""
    from qwb200.engine.engine import EngineOptions
    from qwb200.utils import settings
    prompts = [[(i * 13 + 7) % 900 + 5 for i in range(700)], [(i * 29 + 3) % 900 + 5 for i in range(650)]]
    old = settings.get()
    try:
        settings.set_current(settings.Settings.from_env({}, spill_cache_mb=cache_mb, spill_cache_stats=True))
        res, want = _run(EngineOptions(slots=1, slot_tokens=1024, use_graphs=graphs, prefill_chunk=0), prompts, 12)
        assert res.dm.spill_cache is None
        sp, got = _run(EngineOptions(slots=1, slot_tokens=1024, use_graphs=graphs, prefill_chunk=0, dev_pages=1, host_pages=3), prompts, 12)
    finally:
        settings.set_current(old)
    for (lw, sw), (lg, sg) in zip(want, got):
        assert torch.equal(lw, lg) and sw == sg
    st = sp.dm.spill_cache_stats()
    if cache_mb == 0:
        assert sp.dm.spill_cache is None and st is None
        return
    hits, misses = st
    assert misses > 0 and hits > 0                      # later steps re-read rows that earlier steps fetched
    assert int(sp.dm.spill_cache["ctl"][0]) == 0        # the fill kernel emptied the miss list
    sp.dm.spill_cache_clear()
    assert int(sp.dm.spill_cache["tags"].abs().sum()) == 0


def test_spill_cache_with_conflicts_stays_exact():
    """A cache far smaller than the working set (entries evict each other all the time) changes nothing but speed."""
    from qwb200.engine.engine import EngineOptions
    from qwb200.utils import settings
    prompts = [[(i * 17 + 1) % 900 + 5 for i in range(700)]]
    old = settings.get()
    try:
        settings.set_current(settings.Settings.from_env({}, spill_cache_mb=1, spill_cache_stats=True))
        _, want = _run(EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=0), prompts, 8)
        sp, got = _run(EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=0, dev_pages=1, host_pages=3), prompts, 8)
        assert sp.dm.spill_cache["entries"] >= 64
    finally:
        settings.set_current(old)
    assert torch.equal(want[0][0], got[0][0]) and want[0][1] == got[0][1]


@pytest.mark.parametrize("stage", [True, False])
def test_token_major_prefill_into_spilled_pages_equals_resident(stage):
    """Chunked token-major prefill whose later chunks lie in host pages: with the per-layer staging copy (the attention
    reads the slot's host pages from a device buffer) and without it (the kernel gathers rows from host memory) the logits
    and the following decode steps equal those of a fully resident slot bit for bit.  Slot 1 of 2, so that the slot's
    offset into the host pool is not zero."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.utils import settings
    prompt = [(i * 13 + 7) % 900 + 5 for i in range(700)]

    def run(opts):
        eng = Engine.synthetic(ModelConfig.tiny(), opts, device="cuda:0", exact=True, ple_rows=4096, seed=3)
        lg = eng.prefill(1, prompt).clone()
        t = int(lg.argmax())
        seq = [t]
        for _ in range(6):
            t = eng.decode([1], [t])[0]
            seq.append(t)
        torch.cuda.synchronize()
        eng.dm.check_error()
        return eng, lg, seq
    old = settings.get()
    try:
        settings.set_current(settings.Settings.from_env({}, spill_stage=stage))
        _, lw, sw = run(EngineOptions(slots=2, slot_tokens=1024, use_graphs=False, prefill_chunk=128))
        sp, lg, sg = run(EngineOptions(slots=2, slot_tokens=1024, use_graphs=False, prefill_chunk=128, dev_pages=2, host_pages=6))
    finally:
        settings.set_current(old)
    assert sp.prefiller is not None and (("stage_k" in sp.prefiller.b) == stage)
    assert torch.equal(lw, lg) and sw == sg


def test_spill_pool_reports_its_numa_placement():
    """The host pages come either from the NUMA-placed arena (policy bind / preferred / interleave; the node they landed on
    is read back) or from the CUDA allocator (policy process); both are pinned and hold zeros before first use."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.models.config import ModelConfig
    from qwb200.utils import settings
    old = settings.get()
    try:
        for pol in ("process", "interleave", "auto"):
            settings.set_current(settings.Settings.from_env({}, spill_policy=pol))
            eng = Engine.synthetic(ModelConfig.tiny(), EngineOptions(slots=1, slot_tokens=1024, use_graphs=False, prefill_chunk=0,
                                                                     dev_pages=1, host_pages=3), device="cuda:0", ple_rows=4096)
            info = eng.dm.spill_numa
            assert info is not None and info["policy"] in ("process", "bind", "interleave")
            if pol == "process":
                assert info["policy"] == "process"
            if pol == "interleave" and "fallback" not in info:
                assert info["policy"] == "interleave" and info["node_got"] >= -1
            assert all(t.is_pinned() or "fallback" not in info for t in eng.dm.k_host)
            assert float(eng.dm.k_host[0].float().abs().sum()) == 0.0
            toks = [(i * 13 + 7) % 900 + 5 for i in range(600)]
            eng.prefill(0, toks)
            eng.decode([0], [11])
            torch.cuda.synchronize()
            eng.dm.check_error()
    finally:
        settings.set_current(old)
