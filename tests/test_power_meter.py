"""The power meter's integration against a fake sensor (no GPU, no NVML)."""
import time

from qwb200.utils.power import PowerMeter


def test_constant_power_integrates_to_watts_times_seconds():
    m = PowerMeter(read_watts=lambda: 400.0, period_s=0.01).start()
    time.sleep(0.2)
    r = m.stop()
    assert r["ok"] and abs(r["avg_w"] - 400.0) < 1.0
    assert abs(r["kilojoules"] * 1e3 - 400.0 * r["seconds"]) < 0.05 * 400.0 * r["seconds"]


def test_ramp_uses_trapezoids():
    t0 = time.perf_counter()
    m = PowerMeter(read_watts=lambda: 1000.0 * (time.perf_counter() - t0), period_s=0.005).start()
    time.sleep(0.2)
    r = m.stop()
    assert abs(r["avg_w"] - 500.0 * r["seconds"]) < 40.0          # mean of a ramp from 0 is half its end value


def test_without_a_sensor_it_still_times():
    m = PowerMeter(read_watts=None)
    m.read = None
    r = m.start().stop()
    assert r["ok"] is False and r["seconds"] >= 0
