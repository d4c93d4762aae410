"""One-shot scheduler: requests that are answered by a single pipeline call (classification heads, rerankers,
pixel generation), batched by count and by a token budget.

``pipeline.execute(batch) -> {request_id: output}`` must finish every request of the batch. Reference:
max/python/max/serve/scheduler/one_shot_scheduler.py.
"""

from __future__ import annotations

import queue
from collections import deque
from typing import Deque

from ...pipelines.context import GenerationStatus, TextContext, TextGenerationOutput
from .text_generation_scheduler import SchedulerProgress


class OneShotScheduler:
    def __init__(self, pipeline, request_queue=None, response_queue=None, cancel_queue=None, max_batch_size: int = 32,
                 max_batch_tokens: int = 0):
        self.pipeline = pipeline
        self.request_queue = request_queue if request_queue is not None else queue.SimpleQueue()
        self.response_queue = response_queue if response_queue is not None else queue.SimpleQueue()
        self.cancel_queue = cancel_queue if cancel_queue is not None else queue.SimpleQueue()
        self.max_batch_size, self.max_batch_tokens = max_batch_size, max_batch_tokens
        self.pending: Deque[TextContext] = deque()
        self.total_batches = 0

    def add_request(self, ctx: TextContext) -> None:
        self.request_queue.put_nowait(ctx)

    @staticmethod
    def _drain(q) -> list:
        out = []
        while True:
            try:
                out.append(q.get_nowait())
            except Exception:  # noqa: BLE001  (queue.Empty or a transport's own empty signal)
                return out

    def run_iteration(self) -> SchedulerProgress:
        self.pending.extend(self._drain(self.request_queue))
        for rid in self._drain(self.cancel_queue):
            for c in [c for c in self.pending if c.request_id == rid]:
                self.pending.remove(c)
                self.response_queue.put_nowait({rid: TextGenerationOutput(rid, [], GenerationStatus.CANCELLED)})
        if not self.pending:
            return SchedulerProgress.NO_PROGRESS
        batch, tokens = [], 0
        while self.pending and len(batch) < self.max_batch_size:
            n = self.pending[0].tokens.prompt_len
            if batch and self.max_batch_tokens and tokens + n > self.max_batch_tokens:
                break
            batch.append(self.pending.popleft())
            tokens += n
        outputs = self.pipeline.execute(batch)
        missing = [c.request_id for c in batch if c.request_id not in outputs]
        if missing:
            raise RuntimeError(f"one-shot pipeline left requests unanswered: {missing}")
        self.response_queue.put_nowait(outputs)
        self.total_batches += 1
        return SchedulerProgress.MADE_PROGRESS
