"""Embeddings scheduler: batches pending embedding requests by a token budget and answers each with
one pooled vector. It runs inside the same worker loop as token generation (between generation steps),
so a server can expose both routes from one model.

Reference: max/python/max/serve/scheduler/embeddings_scheduler.py and
max/python/max/pipelines/lib/embeddings_pipeline.py.
"""

from __future__ import annotations

from collections import deque
from typing import Callable, Deque

from ...pipelines.context import EmbeddingsOutput, TextContext


class EmbeddingsScheduler:
    def __init__(self, encode_fn: Callable, response_queue, max_batch_tokens: int = 8192, max_batch_size: int = 64):
        """``encode_fn(token_lists, pooling) -> tensor [n, dim]`` (e.g. ``Llama3Model.encode``)."""
        self.encode_fn, self.response_queue = encode_fn, response_queue
        self.max_batch_tokens, self.max_batch_size = max_batch_tokens, max_batch_size
        self.pending: Deque[TextContext] = deque()
        self.total_batches = 0

    def enqueue(self, ctx: TextContext) -> None:
        self.pending.append(ctx)

    def cancel(self, request_id: str) -> bool:
        for c in list(self.pending):
            if c.request_id == request_id:
                self.pending.remove(c)
                return True
        return False

    def run_iteration(self) -> int:
        """Encode one batch; returns the number of requests answered."""
        if not self.pending:
            return 0
        pooling = self.pending[0].pooling
        batch, tokens = [], 0
        while self.pending and len(batch) < self.max_batch_size and self.pending[0].pooling == pooling:
            n = self.pending[0].tokens.prompt_len
            if batch and tokens + n > self.max_batch_tokens:
                break
            batch.append(self.pending.popleft())
            tokens += n
        vecs = self.encode_fn([c.tokens.all.tolist() for c in batch], pooling).cpu().tolist()
        self.response_queue.put_nowait({c.request_id: EmbeddingsOutput(c.request_id, v, c.tokens.prompt_len)
                                        for c, v in zip(batch, vecs)})
        self.total_batches += 1
        return len(batch)
