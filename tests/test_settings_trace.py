"""Settings parsing / validation and the env-gated tracers (no GPU)."""
import pytest


def test_settings_from_env_aliases_validation_and_unknowns():
    from qwb200.utils.settings import Settings
    s = Settings.from_env({"QW_TRACE": "1", "QW_SLOTS": "65536,8192", "QW_KV_SPILL": "on", "QW_DECODE_SHARE": "0.5", "QW_PREFILL_CHUNK": "2048",
                           "QW_HOST_CACHE_GB": "16", "QW_COMM_SPLIT": "3", "QW_NOT_A_THING": "x", "HOME": "/root"}, prefill_piece=1024)
    assert s.trace and s.kv_spill and s.slots == [65536, 8192] and s.decode_share == 0.5 and s.prefill_chunk == 2048
    assert s.prefill_piece == 1024 and s.host_cache_gb == 16.0 and s.unknown == ["QW_NOT_A_THING"]
    # the reference's spill variables: a per-slot list of tokens beyond the device part, and a switch that forces spill off
    t = Settings.from_env({"QW_SLOT_SPILL": "0,131072", "QW_SPILL": "0", "QW_SLOT_MAX_TOKENS": "524288"})
    assert t.slot_spill == [0, 131072] and t.spill is False and t.slot_max_tokens == 524288 and not t.unknown
    assert Settings.from_env({}).spill is True and Settings.from_env({}).slot_spill == []
    d = s.describe()
    assert "trace=True" in d and "QW_NOT_A_THING" in d and "stuck_seconds" not in d
    assert "all defaults" in Settings.from_env({}).describe()
    for bad in ({"QW_PREFILL_CHUNK": "1000"}, {"QW_DECODE_SHARE": "0"}, {"QW_TRACE": "maybe"}, {"QW_SLOTS": "12"}, {"QW_SPILL_POLICY": "x"},
                {"QW_SPEC_MAX_ROWS": "64"}, {"QW_SLOT_SPILL": "100"}, {"QW_SLOT_MAX_TOKENS": "1000"}):
        with pytest.raises(ValueError):
            Settings.from_env(bad)
    with pytest.raises(ValueError):
        Settings.from_env({}, no_such_option=1)
    env = {}
    Settings.from_env({"QW_MEDIA_FETCH": "0"}).export_env(env)
    assert env["QW_MEDIA_FETCH"] == "0" and env["QW_MEDIA_ALLOW_PRIVATE"] == "0"


def test_tracers_are_silent_when_off_and_aggregate_when_on():
    from qwb200.utils.trace import PhaseTrace, StepTrace
    lines = []
    off = StepTrace(False, log=lines.append)
    for _ in range(100):
        off.begin(); off.launched(); off.enqueued(); off.end(1)
    assert lines == []
    on = StepTrace(True, every=3, log=lines.append)
    for _ in range(7):
        on.begin(); on.launched(); on.enqueued(); on.end(2)
    assert len(lines) == 2 and "rows=2" in lines[0] and "over 3 steps" in lines[0]
    p = PhaseTrace(True, "generate", every=2, log=lines.append)
    for _ in range(2):
        p.start(); p.mark("draft"); p.mark("verify"); p.count("fallbacks"); p.finish()
    assert "draft" in lines[-1] and "verify" in lines[-1] and "fallbacks=2" in lines[-1]
