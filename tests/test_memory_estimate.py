"""Pre-load memory estimate: weights against the sizes the engine reported after loading the full model, the state's
arithmetic, the refusals (device, host) and the wait for a busy GPU - all on CPU."""
import pytest

from qwb200.engine import memory_estimate as ME
from qwb200.models.config import ModelConfig

GB = 1 << 30


def test_weight_estimate_matches_the_loaded_sizes():
    cfg = ModelConfig.full()
    for ranks, loaded_gb in ((1, 72.2), (2, 36.8), (4, 19.1), (8, 10.3)):          # decimal GB logged by the benchmark after loading
        est = ME.weight_bytes(cfg, ranks) / 1e9
        assert abs(est / loaded_gb - 1) < 0.03, (ranks, est)


def test_state_and_spill_arithmetic():
    cfg = ModelConfig.full()
    # one token of KV on one GPU: 13 layers (12 QSA + the MTP head) x K and V x 2 heads x 256 x bf16
    a = ME.state_bytes(cfg, 1, 1, 256, None, 32, False)
    b = ME.state_bytes(cfg, 1, 1, 512, None, 32, False)
    per_token = (b - a) / 256
    assert per_token == 13 * 2 * 2 * 256 * 2 + 13 * 128 * 2 / 4                     # + a compressed key per 4 tokens
    # six slots of 131,072 tokens: ~21 GB of KV, all resident; with three quarters spilled the device keeps a quarter of it
    full = ME.estimate(cfg, 1, slots=6, slot_tokens=131072)
    spilled = ME.estimate(cfg, 1, slots=6, slot_tokens=131072, dev_pages=6 * 128, host_pages=6 * 384)
    kv_gb = 6 * 131072 * 13 * 2 * 2 * 256 * 2 / GB
    assert abs((full["state_gb"] - spilled["state_gb"]) - 0.75 * kv_gb) < 1e-6 and abs(spilled["host_kv_gb"] - 0.75 * kv_gb) < 1e-6
    assert 90 < full["device_gb"] < 110 and full["host_kv_gb"] == 0
    # eight ranks: a KV head lives on four ranks, each stores one head; the recurrent state splits by heads
    e8 = ME.estimate(cfg, 8, slots=4, slot_tokens=131072)
    assert e8["weights_gb"] < 10 and e8["device_gb"] < 30


def test_check_refuses_with_the_numbers():
    cfg = ModelConfig.full()
    ok = ME.estimate(cfg, 1, slots=6, slot_tokens=131072)
    ME.check(ok, 178 * GB, host_available=500 * GB)
    big = ME.estimate(cfg, 1, slots=16, slot_tokens=524288)
    with pytest.raises(ValueError, match=r"does not fit the GPU: weights 6\d\.\d GB \+ slots \d+\.\d GB"):
        ME.check(big, 178 * GB)
    sp = ME.estimate(cfg, 1, slots=6, slot_tokens=524288, dev_pages=6 * 128, host_pages=6 * (2048 - 128))
    ME.check(sp, 178 * GB, host_available=200 * GB)
    with pytest.raises(ValueError, match="pinned host memory"):
        ME.check(sp, 178 * GB, host_available=64 * GB)
    with pytest.raises(ValueError, match="pinned host memory"):
        ME.check(sp, 178 * GB, host_available=200 * GB, local_ranks=4)              # four ranks on this host pin four pools
    tiny = ME.estimate(ModelConfig.tiny(), 1, slots=3, slot_tokens=4096)
    ME.check(tiny, 178 * GB, host_available=ME.host_available_bytes())
    assert ME.host_available_bytes("/no/such/file") is None


def test_wait_for_a_busy_device():
    now = [0.0]
    frees = [10 * GB, 20 * GB, 170 * GB]
    logs = []

    def info():
        return frees[min(int(now[0] // 5), 2)], 178 * GB

    def sleep(s):
        now[0] += s
    assert ME.wait_for_device(info, 600, logs.append, sleep=sleep, clock=lambda: now[0]) is True
    assert now[0] == 10 and "in use" in logs[0] and "free after 10 s" in logs[1]
    now[0], logs[:] = 0.0, []
    assert ME.wait_for_device(lambda: (10 * GB, 178 * GB), 12, logs.append, sleep=sleep, clock=lambda: now[0]) is False
    assert now[0] == 15 and "still busy" in logs[-1]
    logs[:] = []
    assert ME.wait_for_device(lambda: (175 * GB, 178 * GB), 600, logs.append) is True and not logs       # free at once: not a word


def test_open_runs_the_preflight_before_loading(monkeypatch):
    """build_ops: the estimate is made and checked before the engine is built; a configuration that cannot fit is refused
    without loading anything."""
    import torch
    from qwb200 import capi_impl
    from qwb200.engine.engine import Engine
    from qwb200.utils import settings

    class Reached(Exception):
        pass

    def no_engine(*a, **kw):
        raise Reached()
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda d=None: (170 * GB, 178 * GB))
    monkeypatch.setattr(Engine, "synthetic", staticmethod(no_engine))
    try:
        with pytest.raises(Reached):
            capi_impl.build_ops({"synthetic": "tiny", "slots": [4096, 4096], "vision": False}, 0, 1, 0)
        with pytest.raises(ValueError, match="does not fit the GPU"):
            capi_impl.build_ops({"synthetic": "full", "slots": [524288] * 16, "vision": False}, 0, 1, 0)
        monkeypatch.setenv("QW_VRAM_CHECK", "0")
        with pytest.raises(Reached):                                                  # the check can be switched off
            capi_impl.build_ops({"synthetic": "full", "slots": [524288] * 16, "vision": False}, 0, 1, 0)
    finally:
        settings.set_current(None)
