"""ClockSampler against a fake NVML module: samples arrive during a short region, reason bits are
decoded, and only read-only NVML calls are made."""
import sys
import time
import types


def _fake_nvml(calls, bits):
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1

    def rec(name, value):
        def f(*a):
            calls.append(name)
            return value
        return f

    m.nvmlInit = rec("nvmlInit", None)
    m.nvmlShutdown = rec("nvmlShutdown", None)
    m.nvmlDeviceGetHandleByIndex = rec("nvmlDeviceGetHandleByIndex", object())
    m.nvmlDeviceGetHandleByUUID = rec("nvmlDeviceGetHandleByUUID", object())
    m.nvmlDeviceGetClockInfo = rec("nvmlDeviceGetClockInfo", 1350)
    m.nvmlDeviceGetMaxClockInfo = rec("nvmlDeviceGetMaxClockInfo", 1965)
    m.nvmlDeviceGetPowerUsage = rec("nvmlDeviceGetPowerUsage", 987000)
    m.nvmlDeviceGetCurrentClocksEventReasons = rec("nvmlDeviceGetCurrentClocksEventReasons", bits)
    return m


def test_sampler_reads_nvml_during_a_short_region(monkeypatch):
    calls = []
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(calls, 0x4 | 0x20))
    from unified_ccl_b200.utils.timing import ClockSampler

    with ClockSampler(0, period_ms=1) as c:
        time.sleep(0.03)
    s = c.summary()
    assert s["samples"] >= 3
    assert s["sm_mhz"] == 1350.0 and s["sm_max_mhz"] == 1965.0
    assert s["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]
    # nothing but reads: no call that sets clocks, power limits or modes
    assert not [n for n in calls if "Set" in n or "Reset" in n or "Lock" in n]


def test_sampler_without_nvml_or_gpu_does_not_fail(monkeypatch):
    monkeypatch.setitem(sys.modules, "pynvml", None)  # import pynvml -> ImportError
    from unified_ccl_b200.utils.timing import ClockSampler

    with ClockSampler(0) as c:
        time.sleep(0.01)
    assert c.summary()["samples"] >= 0
