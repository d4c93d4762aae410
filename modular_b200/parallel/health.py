"""Host-side failure detection for multi-process (one process per GPU) runs.

Every rank publishes a heartbeat counter and its state in the rendezvous store; before each step a
rank calls ``check()``, which raises :class:`PeerFailure` when a peer announced that it is leaving
(exception, shutdown) or stopped beating for longer than ``timeout_s``. Ranks leave only between
steps, with none of their kernels in flight, so a survivor never launches a kernel that would wait for
a dead peer; kernels that wait on peers have bounded waits anyway and report through the device error
word (``ops.check_device_error``), which ``check()`` also folds in when given.

Reference: the heartbeat watcher of the serving process (max/python/max/serve/process_control.py:239)
and the decode-side stall watchdog (serve/scheduler/decode_scheduler.py:669-686).
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class RankHealth:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 5.0,
                 prefix: str = "mb200/health", startup_timeout_s: float = 120.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._beat = 0
        # (last beat value, time it changed); -1 = the peer has not been seen beating yet (still starting)
        self._seen = {r: (-1, time.monotonic()) for r in range(world) if r != rank}
        self.startup_timeout = startup_timeout_s
        self.store.set(self._k(rank, "state"), "alive")
        self.store.set(self._k(rank, "beat"), "0")
        self._thread = threading.Thread(target=self._loop, name="rank-health", daemon=True)
        self._thread.start()

    def _k(self, rank: int, what: str) -> str:
        return f"{self.prefix}/{rank}/{what}"

    def _loop(self) -> None:
        while not self._stop.wait(self.interval):
            self._beat += 1
            try:
                self.store.set(self._k(self.rank, "beat"), str(self._beat))
            except Exception:  # noqa: BLE001  (store gone: the job is ending)
                return

    def leave(self, reason: str = "shutdown") -> None:
        """Announce departure (call between steps, before exiting or re-raising)."""
        self._stop.set()
        try:
            self.store.set(self._k(self.rank, "state"), f"left:{reason}")
        except Exception:  # noqa: BLE001
            pass

    def check(self, device_error: Optional[Callable[[], None]] = None) -> None:
        """Raise PeerFailure if any peer left or went silent; optionally also surface device-side timeouts."""
        now = time.monotonic()
        for r in list(self._seen):
            last_beat, last_t = self._seen[r]
            try:
                if last_beat < 0 and not self.store.check([self._k(r, "beat")]):
                    if now - last_t > self.startup_timeout:
                        raise PeerFailure(r, f"never started ({now - last_t:.0f} s)")
                    continue
                state = self.store.get(self._k(r, "state")).decode()
                beat = int(self.store.get(self._k(r, "beat")).decode())
            except PeerFailure:
                raise
            except Exception as e:  # noqa: BLE001
                raise PeerFailure(r, f"health record unreadable ({e!r})") from e
            if state.startswith("left"):
                raise PeerFailure(r, state)
            if beat != last_beat:
                self._seen[r] = (beat, now)
            elif now - last_t > self.timeout:
                raise PeerFailure(r, f"no heartbeat for {now - last_t:.1f} s")
        if device_error is not None:
            device_error()

    def guard(self):
        """Context manager for a rank's main loop: a rank that raises tells its peers before it dies."""
        health = self

        class _Guard:
            def __enter__(self_inner):
                return health

            def __exit__(self_inner, exc_type, exc, tb):
                health.leave("shutdown" if exc_type is None else f"{exc_type.__name__}: {exc}")
                return False

        return _Guard()
