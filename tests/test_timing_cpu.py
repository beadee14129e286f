"""Clock sampling and latency statistics of the benchmarks, without a GPU: NVML is replaced by a fake module that
plays back a clock / reason / power trace, nvidia-smi by canned CSV lines."""
import sys
import time
import types

from ooverlap_b200.utils import timing


def test_percentiles_nearest_rank():
    assert timing.percentiles([])["n"] == 0 and timing.percentiles([])["p50"] is None
    p = timing.percentiles([float(i) for i in range(1, 101)])
    assert p["n"] == 100 and p["p50"] in (50.0, 51.0) and p["p90"] in (90.0, 91.0) and p["p99"] in (99.0, 100.0)
    assert p["mean"] == 50.5
    assert timing.percentiles([7.0]) == {"p50": 7.0, "p90": 7.0, "p99": 7.0, "mean": 7.0, "n": 1}


def _fake_nvml(trace):
    """A stand-in for pynvml that returns (MHz, reason bits, milliwatts) from `trace`, the last entry for ever."""
    state = {"i": 0}
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1
    m.nvmlInit = lambda: None
    m.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    m.nvmlDeviceGetHandleByUUID = lambda u: ("handle", u)
    m.nvmlDeviceGetMaxClockInfo = lambda h, c: 1965

    def cur():
        return trace[min(state["i"], len(trace) - 1)]

    def clock(h, c):
        v = cur()[0]
        state["i"] += 1
        return v

    m.nvmlDeviceGetClockInfo = clock
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: cur()[1]
    m.nvmlDeviceGetPowerUsage = lambda h: cur()[2]
    return m


def test_nvml_sampler_summarises_only_the_timed_region(monkeypatch):
    # idle clocks before the region, then a power-capped plateau
    trace = [(345, 0x1, 90_000)] * 3 + [(1350, 0x4, 990_000)] * 10_000
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(trace))
    s = timing.NvmlClockSampler(0, period_ms=1.0)
    assert s.available
    s.start()
    time.sleep(0.03)            # the three idle samples are consumed before the region opens
    s.begin()
    time.sleep(0.06)
    s.end()
    time.sleep(0.01)
    out = s.stop()
    assert out["source"] == "nvml" and out["sm_max_mhz"] == 1965.0
    assert out["samples"] >= 3 and out["samples_total"] > out["samples"]
    assert out["sm_mhz"] == 1350 and out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 990.0


def test_nvml_sampler_reports_thermal_and_hw_slowdown_bits(monkeypatch):
    trace = [(1200, 0x8 | 0x20 | 0x40, 500_000)] * 10_000
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(trace))
    s = timing.NvmlClockSampler(0, period_ms=1.0).start()
    s.begin()
    time.sleep(0.03)
    s.end()
    out = s.stop()
    assert out["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]


def test_nvml_sampler_is_unavailable_without_nvml(monkeypatch):
    broken = types.ModuleType("pynvml")

    def boom():
        raise RuntimeError("no driver")

    broken.nvmlInit = boom
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    s = timing.NvmlClockSampler(0)
    assert not s.available
    assert s.start() is s
    out = s.stop()
    assert out["sm_mhz"] is None and out["samples"] == 0 and out["reasons"] == []


def test_nvidia_smi_lines_are_parsed():
    s = timing.ClockSampler(0, period_ms=1)
    s._lines = [
        "0, 1965, 1965, 310.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
        "0, 1350, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "0, 1340, 1965, 999.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "garbage",
        "0, [N/A], 1965, 1.0, 0x0, Not Active, Not Active, Not Active, Not Active",
    ]
    out = s.stop()  # no process was started: only the parsing runs
    assert out == {"sm_mhz": 1350.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
