"""CPython garbage collector and host allocator housekeeping for the serving processes.

A cyclic collection stops the scheduler loop of the model worker: with millions of long-lived objects (weights
metadata, cache bookkeeping, captured graphs) a full collection costs tens of milliseconds, which shows up as a
spike in the time between tokens. Three tools:

* :func:`freeze_startup_heap` - after start-up and warm-up, move everything alive into the permanent generation
  (``gc.freeze``): later collections only look at what the serving loop allocates.
* :class:`GCPauseMonitor` - a ``gc.callbacks`` hook that measures every collection, feeds the
  ``maxserve_gc_pause_ms`` histogram and logs the slow ones (optionally with the most common types of the
  generation, which costs a walk over it).
* :func:`trim_host_heap` - hand free pages of the C allocator back to the operating system after the start-up
  peak (``malloc_trim``; a no-op where libc has none).

Reference: max/python/max/serve/telemetry/gc_utils.py (GCDebugger :28, freeze_gc_heap :126,
_release_free_host_memory :151), called from pipelines/model_worker.py:472-488.
"""

from __future__ import annotations

import ctypes
import gc
import logging
import time
from collections import Counter
from typing import Optional

logger = logging.getLogger("modular_b200.serve")


class GCPauseMonitor:
    """Callable for ``gc.callbacks``. CPython calls it with ``"start"`` right before and ``"stop"`` right after a
    collection, on the collecting thread and with the GIL held throughout, so one start stamp is enough."""

    def __init__(self, slow_ms: float = 5.0, top_types: int = 0, observe=None):
        self.slow_ms, self.top_types, self.observe = slow_ms, top_types, observe
        self.collections = 0
        self.total_ms = 0.0
        self.max_ms = 0.0
        self._t0 = 0
        self._census: Optional[dict] = None

    def __call__(self, phase: str, info: dict) -> None:
        gen = info.get("generation")
        if gen is None:
            return
        if phase == "start":
            if self.top_types > 0:        # walks the whole generation: only while hunting for what fills the heap
                self._census = dict(Counter(type(o).__qualname__ for o in gc.get_objects(gen)).most_common(self.top_types))
            self._t0 = time.monotonic_ns()
        elif phase == "stop" and self._t0:
            ms = (time.monotonic_ns() - self._t0) / 1e6
            self._t0 = 0
            self.collections += 1
            self.total_ms += ms
            self.max_ms = max(self.max_ms, ms)
            if self.observe is not None:
                try:
                    self.observe(ms)
                except Exception:      # noqa: BLE001 - a metrics failure must not break a collection
                    pass
            if ms >= self.slow_ms:
                logger.info("GC generation %d paused the process for %.2f ms (collected %s)%s", gen, ms,
                            info.get("collected", "?"), f"; most common types: {self._census}" if self._census else "")


def install_gc_monitor(enabled: bool = True, slow_ms: float = 5.0, top_types: int = 0, observe=None):
    """Attaches a :class:`GCPauseMonitor` (once per process, after logging is configured); None when disabled."""
    if not enabled:
        return None
    mon = GCPauseMonitor(slow_ms, top_types, observe)
    gc.callbacks.append(mon)
    return mon


def remove_gc_monitor(mon) -> None:
    if mon is not None and mon in gc.callbacks:
        gc.callbacks.remove(mon)


def freeze_startup_heap() -> int:
    """Collect every generation, then freeze what survived. Returns the size of the permanent generation."""
    for g in (0, 1, 2):
        gc.collect(g)
    gc.freeze()
    return gc.get_freeze_count()


def trim_host_heap() -> bool:
    """``malloc_trim(0)`` where the C library has it. Returns whether it ran."""
    try:
        fn = ctypes.CDLL(None).malloc_trim
    except (OSError, AttributeError):
        return False
    fn.argtypes, fn.restype = [ctypes.c_size_t], ctypes.c_int
    fn(0)
    return True
