"""Host-side pieces of bench.py that need no GPU: the clock sampler (against a fake NVML: nothing of a GPU is read or
set here), the DRAM-traffic table lookup and the rounding of the JSON line."""
import importlib.util
import os
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _fake_nvml(clock_mhz, reasons):
    return types.SimpleNamespace(
        NVML_CLOCK_SM=1,
        nvmlDeviceGetClockInfo=lambda h, c: clock_mhz,
        nvmlDeviceGetMaxClockInfo=lambda h, c: 1965,
        nvmlDeviceGetPowerUsage=lambda h: 500000,
        nvmlDeviceGetCurrentClocksEventReasons=lambda h: reasons,
        nvmlClocksEventReasonHwSlowdown=0x8, nvmlClocksEventReasonHwThermalSlowdown=0x40,
        nvmlClocksEventReasonSwThermalSlowdown=0x20, nvmlClocksEventReasonSwPowerCap=0x4)


def test_clock_sampler_keeps_the_samples_of_the_timed_region():
    b = _bench()
    cs = b.ClockSampler(0)
    cs._nvml_handle = lambda: (_fake_nvml(1950, 0x4), object())
    cs.start()
    time.sleep(0.03)
    cs.mark_begin()
    time.sleep(0.06)
    cs.mark_end()
    time.sleep(0.03)
    r = cs.stop()
    assert r["sm_mhz"] == 1950.0 and r["sm_max_mhz"] == 1965.0 and r["power_w_max"] == 500.0
    assert r["reasons"] == ["sw_power_cap"] and "inside the timed region" in r["sampled"]
    assert 3 <= r["samples"] <= 40          # ~2 ms apart over 60 ms; the 30 ms before and after are left out


def test_clock_sampler_names_every_slowdown_reason():
    b = _bench()
    cs = b.ClockSampler(0)
    cs._nvml_handle = lambda: (_fake_nvml(1200, 0x8 | 0x40 | 0x20), object())
    cs.start()
    cs.mark_begin()
    time.sleep(0.02)
    cs.mark_end()
    r = cs.stop()
    assert r["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]


def test_dram_traffic_table_and_rounding():
    b = _bench()
    assert b.dram_traffic("dw", "llama3-8b-mlp") > 3.0e8
    assert b.dram_traffic("dx", "llama3-8b-mlp") > 1.0e8
    assert b.dram_traffic("no-such-kernel", "llama3-8b-mlp") is None
    assert b.compact({"a": 1.23456789, "b": [float("nan"), 2.0], "c": "s"}) == {"a": 1.2346, "b": [None, 2.0], "c": "s"}
