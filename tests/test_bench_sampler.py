"""bench.py's clock sampler against a fake NVML (read-only queries, no GPU needed)."""
import importlib.util
import pathlib
import sys
import time
import types

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _fake_nvml(reason_bits, clocks):
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1
    m.calls = []
    it = iter(clocks)
    last = [clocks[-1]]

    def clock(_h, _kind):
        try:
            last[0] = next(it)
        except StopIteration:
            pass
        return last[0]
    m.nvmlInit = lambda: m.calls.append("init")
    m.nvmlDeviceGetHandleByUUID = lambda u: (_ for _ in ()).throw(RuntimeError("no such uuid"))
    m.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    m.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    m.nvmlDeviceGetClockInfo = clock
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: reason_bits
    return m


def test_sampler_reads_clocks_and_reasons_from_nvml(monkeypatch):
    bench = _load_bench()
    fake = _fake_nvml(0x4 | 0x1, [1800, 1500, 1500, 1300])      # sw_power_cap + idle bit (ignored)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.ClockSampler(3, "GPU-deadbeef")
    s.start()
    time.sleep(0.15)
    out = s.stop()
    assert out["source"] == "nvml" and out["samples"] >= 3
    assert out["sm_max_mhz"] == 1965.0 and 1300.0 <= out["sm_mhz"] <= 1800.0
    assert out["reasons"] == ["sw_power_cap"]
    assert "init" in fake.calls


def test_sampler_reports_thermal_and_hw_slowdown(monkeypatch):
    bench = _load_bench()
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(0x8 | 0x20 | 0x40, [1000]))
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.06)
    out = s.stop()
    assert out["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]


def test_sampler_without_nvml_or_nvidia_smi_returns_empty(monkeypatch):
    bench = _load_bench()
    broken = types.ModuleType("pynvml")
    broken.nvmlInit = lambda: (_ for _ in ()).throw(RuntimeError("no driver"))
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    monkeypatch.setenv("PATH", "/nonexistent")
    s = bench.ClockSampler(0)
    s.start()
    out = s.stop()
    assert out["samples"] == 0 and out["sm_mhz"] is None and out["reasons"] == []
