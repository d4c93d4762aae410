"""Subprocess supervision: spawn, wait until ready, watch a heartbeat, cancel as a group.

Reference: max/python/max/serve/process_control.py:152 ``ProcessManager`` (``ready`` :201,
``watch_heartbeat`` :239), ``subprocess_manager`` :267.
"""

from __future__ import annotations

import asyncio
import contextlib
import multiprocessing as mp
import time
from typing import Callable, Optional


class SubprocessExit(RuntimeError):
    """The supervised process ended (or stopped beating) while the server still needed it."""


class ProcessManager:
    def __init__(self, name: str, target: Callable, args: tuple = (), ctx=None, daemon: bool = True):
        """``daemon=False`` for a child that starts processes of its own (a daemonic process may not); such a
        child is stopped by :meth:`shutdown`, also at interpreter exit."""
        self.name = name
        self.ctx = ctx or mp.get_context("spawn")
        self.ready_event = self.ctx.Event()
        self.alive_event = self.ctx.Event()
        self.stop_event = self.ctx.Event()
        self.process = self.ctx.Process(target=target, name=name, daemon=daemon,
                                        args=(*args, self.ready_event, self.alive_event, self.stop_event))
        if not daemon:
            import atexit

            atexit.register(self.shutdown, 1.0)

    def start(self) -> None:
        self.process.start()

    async def ready(self, timeout_s: float) -> None:
        """Return when the child signalled readiness; raise if it died or timed out first."""
        t0 = time.monotonic()
        while not self.ready_event.is_set():
            if not self.process.is_alive():
                raise SubprocessExit(f"{self.name} exited with code {self.process.exitcode} before it was ready")
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError(f"{self.name} was not ready within {timeout_s:.0f} s")
            await asyncio.sleep(0.05)

    async def watch_heartbeat(self, fail_after_s: float, poll_s: float = 0.5) -> None:
        """Raise SubprocessExit when the child stops setting ``alive_event`` for ``fail_after_s``."""
        last = time.monotonic()
        while True:
            await asyncio.sleep(poll_s)
            if self.alive_event.is_set():
                self.alive_event.clear()
                last = time.monotonic()
            elif time.monotonic() - last > fail_after_s:
                raise SubprocessExit(f"{self.name} missed its heartbeat for {fail_after_s:.0f} s")
            if not self.process.is_alive():
                raise SubprocessExit(f"{self.name} exited with code {self.process.exitcode}")

    async def watch_exit(self, poll_s: float = 0.2) -> None:
        while self.process.is_alive():
            await asyncio.sleep(poll_s)
        raise SubprocessExit(f"{self.name} exited with code {self.process.exitcode}")

    def shutdown(self, grace_s: float = 5.0) -> None:
        self.stop_event.set()
        if self.process.pid is None:
            return
        if self.process.is_alive():
            self.process.join(grace_s)
        if self.process.is_alive():
            self.process.terminate()
            self.process.join(grace_s)
        if self.process.is_alive():
            self.process.kill()


@contextlib.asynccontextmanager
async def subprocess_manager(name: str, target: Callable, args: tuple = (), ready_timeout_s: float = 1200.0,
                             use_heartbeat: bool = False, health_fail_s: float = 60.0, daemon: bool = True):
    """Start ``target`` in a spawned process, wait until ready, yield (manager, watcher task).

    The watcher task fails with SubprocessExit if the child dies (or stops beating); callers
    await it alongside the server so a worker crash brings the server down."""
    pm = ProcessManager(name, target, args, daemon=daemon)
    pm.start()
    watcher: Optional[asyncio.Task] = None
    try:
        await pm.ready(ready_timeout_s)
        watcher = asyncio.create_task(pm.watch_heartbeat(health_fail_s) if use_heartbeat else pm.watch_exit())
        yield pm, watcher
    finally:
        if watcher is not None:
            watcher.cancel()
            with contextlib.suppress(BaseException):
                await watcher
        pm.shutdown()
