"""Proxy the API process uses to talk to the model worker: submit, stream, cancel."""

from __future__ import annotations

import asyncio
import queue
from dataclasses import dataclass
from typing import Any, AsyncIterator, Optional


class RequestQueueFull(RuntimeError):
    """More requests are pending than ``max_queue_size`` allows (mapped to HTTP 429)."""


class WorkerGone(RuntimeError):
    """The model worker process behind a proxy has exited (mapped to HTTP 503)."""


@dataclass
class WorkerQueues:
    request: Any
    response: Any
    cancel: Any


class ModelWorkerProxy:
    """Fan-out of worker responses to per-request asyncio queues."""

    def __init__(self, queues: WorkerQueues, max_queue_size: int = 0, poll_s: float = 0.001):
        self.queues = queues
        self.max_queue_size = max_queue_size
        self.poll_s = poll_s
        self._streams: dict[str, asyncio.Queue] = {}
        self._task: Optional[asyncio.Task] = None
        self.dead: Optional[str] = None      # set by abort_all

    def start(self) -> None:
        if self._task is None:
            self._task = asyncio.create_task(self._response_worker())

    async def stop(self) -> None:
        if self._task is not None:
            self._task.cancel()
            try:
                await self._task
            except BaseException:  # noqa: BLE001
                pass
            self._task = None

    @property
    def pending(self) -> int:
        return len(self._streams)

    async def _response_worker(self) -> None:
        idle = 0
        while True:
            got = False
            while True:
                try:
                    batch = self.queues.response.get_nowait()
                except queue.Empty:
                    break
                except Exception:  # noqa: BLE001
                    break
                got = True
                for rid, out in batch.items():
                    q = self._streams.get(rid)
                    if q is not None:
                        q.put_nowait(out)
            idle = 0 if got else min(idle + 1, 20)
            await asyncio.sleep(0 if got else self.poll_s * (1 + idle))

    async def stream(self, ctx) -> AsyncIterator:
        """Submit ``ctx`` and yield TextGenerationOutput chunks until the final one."""
        if self.dead is not None:
            raise WorkerGone(self.dead)
        if self.max_queue_size and len(self._streams) >= self.max_queue_size:
            raise RequestQueueFull(f"{len(self._streams)} requests pending (limit {self.max_queue_size})")
        q: asyncio.Queue = asyncio.Queue()
        self._streams[ctx.request_id] = q
        try:
            self.queues.request.put_nowait(ctx)
            while True:
                out = await q.get()
                yield out
                if out.is_done:
                    return
        finally:
            still = self._streams.pop(ctx.request_id, None)
            if still is not None and not ctx_done(still):
                try:
                    self.queues.cancel.put_nowait(ctx.request_id)
                except Exception:  # noqa: BLE001
                    pass

    def abort_all(self, message: str) -> None:
        """The worker behind this proxy is gone: every waiting request ends with an error, and requests that arrive
        later are refused at once instead of waiting for an answer that cannot come."""
        from ...pipelines.context import GenerationStatus, TextGenerationOutput

        self.dead = message
        for rid, q in list(self._streams.items()):
            q.put_nowait(TextGenerationOutput(rid, [], GenerationStatus.ERROR, None, message))

    def cancel(self, request_id: str) -> None:
        self.queues.cancel.put_nowait(request_id)
        q = self._streams.get(request_id)
        if q is not None:
            from ...pipelines.context import GenerationStatus, TextGenerationOutput

            q.put_nowait(TextGenerationOutput(request_id, [], GenerationStatus.CANCELLED))


def ctx_done(q: asyncio.Queue) -> bool:
    """True when the stream ended normally (nothing left to cancel on the worker)."""
    return getattr(q, "_finished_normally", False)


class ReplicaRouter:
    """Data-parallel replicas behind one proxy interface: every replica is a full model worker (own
    GPU, own scheduler and KV cache); a request goes to the replica with the fewest requests in
    flight, ties broken round-robin, and stays there (its KV cache lives on that replica).

    Reference: max/python/max/serve/scheduler/batch_constructor/text_batch_constructor.py:566-594
    (least-loaded replica assignment) and the data_parallel_degree setting of the model config.
    """

    def __init__(self, proxies):
        if not proxies:
            raise ValueError("at least one replica is needed")
        self.proxies = list(proxies)
        self._rr = 0
        self.assigned = [0] * len(self.proxies)      # requests ever routed to each replica

    def start(self) -> None:
        for p in self.proxies:
            p.start()

    async def stop(self) -> None:
        for p in self.proxies:
            await p.stop()

    @property
    def pending(self) -> int:
        return sum(p.pending for p in self.proxies)

    @property
    def dead(self) -> Optional[str]:
        """Set once every replica is gone (one dead replica only stops receiving requests)."""
        gone = [p.dead for p in self.proxies]
        return gone[0] if all(gone) else None

    def pick(self) -> int:
        n = len(self.proxies)
        alive = [i for i in range(n) if self.proxies[i].dead is None] or list(range(n))
        best = min(alive, key=lambda i: (self.proxies[i].pending, (i - self._rr) % n))
        self._rr = (best + 1) % n
        return best

    async def stream(self, ctx):
        i = self.pick()
        self.assigned[i] += 1
        async for out in self.proxies[i].stream(ctx):
            yield out

    def cancel(self, request_id: str) -> None:
        for p in self.proxies:
            if request_id in p._streams:
                p.cancel(request_id)
