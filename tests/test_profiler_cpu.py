"""Profiler: ranges are free when disabled, recorded when enabled; the GPU recorder against a fake NVML."""

import json
import time
import types

from modular_b200 import profiler


def test_tracer_and_traced_record_ranges():
    calls = []

    @profiler.traced
    def work(x):
        calls.append(x)
        return x + 1

    profiler.enable(False)
    assert work(1) == 2
    profiler.enable(True)
    try:
        with profiler.Tracer("outer"):
            assert work(2) == 3
            t = profiler.Tracer()
            t.next("phase-a")
            t.next("phase-b")
            t.close()
        trace = json.loads(profiler.dump_chrome_trace())
    finally:
        profiler.enable(False)
    names = {e.get("name") for e in (trace if isinstance(trace, list) else trace.get("traceEvents", []))}
    assert {"outer", "phase-a", "phase-b"} <= names and any("work" in (n or "") for n in names)
    assert calls == [1, 2]


def test_gpu_recorder_with_fake_nvml():
    fake = types.SimpleNamespace(NVML_CLOCK_SM=1, n=0)
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: i
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    fake.nvmlDeviceGetClockInfo = lambda h, k: 1300
    fake.nvmlDeviceGetPowerUsage = lambda h: 950_000
    fake.nvmlDeviceGetMemoryInfo = lambda h: types.SimpleNamespace(used=10 << 30)
    fake.nvmlDeviceGetUtilizationRates = lambda h: types.SimpleNamespace(gpu=99)
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4
    with profiler.GpuRecorder(0, interval_s=0.01, nvml=fake) as rec:
        time.sleep(0.1)
    s = rec.summary()
    assert s["samples"] >= 2 and s["sm_mhz"] == 1300 and s["sm_max_mhz"] == 1965
    assert s["reasons"] == ["sw_power_cap"] and s["power_w"] == 950.0 and s["error"] is None
