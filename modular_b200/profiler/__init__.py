"""Profiling helpers: NVTX ranges, a host-side Chrome trace, and a background GPU recorder.

* ``Tracer`` / ``@traced``: named ranges. They cost one attribute check unless profiling is enabled
  (``MODULAR_ENABLE_PROFILING=1`` or :func:`enable`). Enabled ranges go to NVTX (when CUDA is present,
  so Nsight tools show them) and to the native Chrome-trace sink of the C++ runtime when it is loaded.
* ``GpuRecorder``: samples clocks, power, utilisation and memory through NVML on a background thread
  (read-only queries) and reports medians plus the set of throttle reasons seen, which is what the
  serving benchmark attaches to its results.

Reference: max/python/max/profiler/tracing.py (``Tracer``, ``traced``), profiler/gpu/bgrec.py:282
(background recorder), profiler/gpu/_nvml.py.
"""

from __future__ import annotations

import functools
import os
import statistics
import threading
import time
from typing import Callable, Optional

_ENABLED = os.environ.get("MODULAR_ENABLE_PROFILING", os.environ.get("MB200_ENABLE_PROFILING", "0")) not in ("", "0")


def enable(on: bool = True) -> None:
    """Turn ranges on or off (also switches the native Chrome-trace sink when it is loaded)."""
    global _ENABLED
    _ENABLED = on
    nat = _native()
    if nat is not None:
        nat.prof_enable(on)


def dump_chrome_trace(clear: bool = True) -> str:
    """JSON text of the host ranges recorded so far (load it in chrome://tracing or Perfetto)."""
    nat = _native()
    return nat.prof_dump_chrome_trace(clear) if nat is not None else "[]"


def is_enabled() -> bool:
    return _ENABLED


def _nvtx():
    try:
        import torch
        if torch.cuda.is_available():
            return torch.cuda.nvtx
    except Exception:  # noqa: BLE001
        pass
    return None


def _native():
    try:
        from .._native import lib
        L = lib(required=False)
        return L if L is not None and hasattr(L, "prof_push") else None
    except Exception:  # noqa: BLE001
        return None


class Tracer:
    """``with Tracer("prefill"):`` or ``t = Tracer(); t.next("a"); t.next("b"); t.close()``."""

    __slots__ = ("_name", "_open", "_nvtx", "_nat")

    def __init__(self, name: Optional[str] = None):
        self._name, self._open = name, False
        self._nvtx = self._nat = None

    def _push(self, name: str) -> None:
        if not _ENABLED:
            return
        self._nvtx, self._nat = _nvtx(), _native()
        if self._nvtx is not None:
            self._nvtx.range_push(name)
        if self._nat is not None:
            self._nat.prof_push(name)
        self._open = True

    def _pop(self) -> None:
        if not self._open:
            return
        if self._nvtx is not None:
            self._nvtx.range_pop()
        if self._nat is not None:
            self._nat.prof_pop()
        self._open = False

    def __enter__(self):
        if self._name is not None:
            self._push(self._name)
        return self

    def __exit__(self, *exc):
        self._pop()
        return False

    def next(self, name: str) -> None:
        self._pop()
        self._push(name)

    def close(self) -> None:
        self._pop()


def traced(fn: Optional[Callable] = None, *, message: Optional[str] = None):
    """Decorator: wrap the call in a range named after the function (or ``message``)."""
    def deco(f):
        label = message or f.__qualname__

        @functools.wraps(f)
        def wrapper(*a, **kw):
            if not _ENABLED:
                return f(*a, **kw)
            with Tracer(label):
                return f(*a, **kw)
        return wrapper
    return deco(fn) if fn is not None else deco


_REASON_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}


class GpuRecorder:
    """Background NVML sampler. ``nvml`` may be injected (tests use a fake with the pynvml API)."""

    def __init__(self, device_index: int = 0, interval_s: float = 0.2, nvml=None):
        self.index, self.interval = device_index, interval_s
        self._nvml = nvml
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.samples: list = []
        self.error: Optional[str] = None

    def _loop(self) -> None:
        nv = self._nvml
        try:
            if nv is None:
                import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            while not self._stop.is_set():
                mem = nv.nvmlDeviceGetMemoryInfo(h)
                util = nv.nvmlDeviceGetUtilizationRates(h)
                self.samples.append(dict(
                    t=time.time(), sm_mhz=nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                    power_w=nv.nvmlDeviceGetPowerUsage(h) / 1000.0, util=util.gpu, mem_used=mem.used,
                    reasons=int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                    if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                    else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
                self._stop.wait(self.interval)
        except Exception as e:  # noqa: BLE001
            self.error = f"{type(e).__name__}: {e}"

    def __enter__(self):
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, name="gpu-recorder", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        return False

    def summary(self) -> dict:
        if not self.samples:
            return {"samples": 0, "error": self.error}
        busy = [s for s in self.samples if s["util"] > 0] or self.samples
        bits = 0
        for s in busy:
            bits |= s["reasons"]
        reasons = sorted(n for b, n in _REASON_BITS.items() if bits & b and n != "gpu_idle")
        return {"samples": len(self.samples), "sm_mhz": statistics.median(s["sm_mhz"] for s in busy),
                "sm_max_mhz": getattr(self, "max_sm_mhz", None),
                "power_w": round(statistics.median(s["power_w"] for s in busy), 1),
                "mem_used_peak": max(s["mem_used"] for s in self.samples), "reasons": reasons,
                "error": self.error}
