"""Host-side pieces of bench.py that need no GPU: the clock sampler against a fake NVML module."""
import importlib.util
import os
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_sampler_reads_nvml(monkeypatch):
    """The sampler polls NVML from a thread: SM clock, maximum clock and the throttle-reason bit mask; the summary names the
    reasons that were active in any sample and the median clock. Nothing but read-outs is called."""
    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetHandleByPciBusId = lambda s: ("handle", s)
    clocks = iter([1965, 1965, 1800] + [1965] * 10000)
    fake.nvmlDeviceGetClockInfo = lambda h, k: next(clocks)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4  # software power cap
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.05)
    out = s.stop()
    assert out["source"] == "nvml" and out["samples"] >= 3
    assert out["sm_mhz"] == 1965 and out["sm_max_mhz"] == 1965
    assert out["reasons"] == ["sw_power_cap"]
    assert calls == ["init"]


def test_clock_sampler_without_nvml_or_nvidia_smi(monkeypatch):
    """No NVML module and no nvidia-smi binary: the sampler reports that instead of failing the benchmark."""
    monkeypatch.setitem(sys.modules, "pynvml", None)  # import pynvml -> ImportError
    monkeypatch.setenv("PATH", "/nonexistent")
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.start()
    out = s.stop()
    assert out["sm_mhz"] is None and out["reasons"] == ["nvidia-smi unavailable"]
