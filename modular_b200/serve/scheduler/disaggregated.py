"""Disaggregated inference: a prefill engine computes the prompt's KV cache and first token, a decode
engine receives both and generates the rest.

Flow for one request (decode node is the front door):
    decode: reserve KV pages for the prompt -> send PrefillRequest(ctx id, tokens, sampling) to prefill
    prefill: run the prompt through its own engine (chunked as usual) until the first token is
             sampled -> export the request's KV pages -> send PrefillResult(first token, pages)
    decode: import the pages into the reserved ones, append the first token, and schedule the
            request as an ordinary decode (token-generation) request.

``KVTransfer`` moves page tensors between engines: ``LocalTransfer`` (same process, direct copy:
tests and single-node prefill/decode on one GPU pair through peer copies) and ``DistTransfer``
(``torch.distributed`` send/recv: NCCL over NVLink between GPUs, gloo on CPU).
The decode side has a stall watchdog (``decode_stall_timeout_s``: no prefill answer for that long
is a fatal error) and a per-request TTL that frees reservations whose prefill never came back.

Reference: max/python/max/serve/scheduler/decode_scheduler.py:116 (reserve + dispatch, TTL eviction
:458, stall watchdog :669-686), prefill_scheduler.py:85, di_dispatchers.py, and the NIXL transfer
engine pipelines/kv_cache/paged_kv_cache/transfer_engine.py:733.
"""

from __future__ import annotations

import queue
import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ...pipelines.context import SamplingParams, TextContext


@dataclass
class PrefillRequest:
    request_id: str
    tokens: np.ndarray
    sampling_params: SamplingParams
    sent_at: float = field(default_factory=time.monotonic)


@dataclass
class PrefillResult:
    request_id: str
    first_token: int
    n_tokens: int                  # prompt tokens whose KV is in `pages`
    pages: Optional[torch.Tensor]  # [n_pages, kv_dim, layers, heads, page, head_dim] (None with DistTransfer)
    n_pages: int = 0


class KVTransfer:
    def send(self, pages: torch.Tensor, dst: int = 0) -> Optional[torch.Tensor]:
        raise NotImplementedError

    def recv(self, like: torch.Tensor, handle, src: int = 0) -> torch.Tensor:
        raise NotImplementedError


class LocalTransfer(KVTransfer):
    """Both engines live in this process: the page tensor itself is the message (a device-to-device copy
    when the engines sit on different GPUs)."""

    def send(self, pages, dst=0):
        return pages

    def recv(self, like, handle, src=0):
        return handle.to(like.device, non_blocking=True)


class DistTransfer(KVTransfer):
    """torch.distributed point-to-point (NCCL between GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group

    def send(self, pages, dst=0):
        self.dist.send(pages.contiguous(), dst, group=self.group)
        return None

    def recv(self, like, handle, src=0):
        buf = torch.empty_like(like)
        self.dist.recv(buf, src, group=self.group)
        return buf


def export_pages(kv_manager, request_id: str, n_tokens: int) -> torch.Tensor:
    """Copy of the pages holding the first ``n_tokens`` tokens of a request."""
    n = (n_tokens + kv_manager.page_size - 1) // kv_manager.page_size
    idx = torch.as_tensor(kv_manager.blocks_of(request_id)[:n], device=kv_manager.kv.device)
    return kv_manager.kv.index_select(0, idx)


def import_pages(kv_manager, request_id: str, pages: torch.Tensor) -> None:
    idx = torch.as_tensor(kv_manager.blocks_of(request_id)[: pages.shape[0]], device=kv_manager.kv.device)
    kv_manager.kv.index_copy_(0, idx, pages.to(kv_manager.kv.device, kv_manager.kv.dtype))


class PrefillNode:
    """Prefill-only engine: ``llm`` is an :class:`modular_b200.entrypoints.llm.LLM`."""

    def __init__(self, llm, inbox, outbox, transfer: KVTransfer = LocalTransfer()):
        self.llm, self.inbox, self.outbox, self.transfer = llm, inbox, outbox, transfer
        self._live: dict[str, PrefillRequest] = {}
        self.completed = 0

    def run_iteration(self) -> int:
        while True:
            try:
                req: PrefillRequest = self.inbox.get_nowait()
            except queue.Empty:
                break
            sp = SamplingParams(**{**req.sampling_params.__dict__, "max_new_tokens": 1})
            self.llm.add_request(req.tokens, sp, request_id=req.request_id)
            self._live[req.request_id] = req
        if not self.llm.has_unfinished():
            return 0
        done = 0
        # the request's pages are released when it finishes, so export them before the step that ends it
        # would free them: with max_new_tokens == 1 the sequence ends as soon as its first token exists
        self.llm.scheduler.batch_constructor.on_release = self._on_release
        for rec in self.llm.step():
            req = self._live.pop(rec.request_id, None)
            if req is None:
                continue
            pages = self._exported.pop(rec.request_id)
            handle = self.transfer.send(pages)
            self.outbox.put_nowait(PrefillResult(rec.request_id, int(rec.tokens[0]), len(req.tokens), handle,
                                                 pages.shape[0]))
            done += 1
            self.completed += 1
        return done

    _exported: dict = {}

    def _on_release(self, request_id: str, n_tokens: int) -> None:
        if request_id in self._live:
            self._exported[request_id] = export_pages(self.llm.kv, request_id, n_tokens)


class DecodeNode:
    """Decode-only engine in front of a prefill node."""

    def __init__(self, llm, to_prefill, from_prefill, transfer: KVTransfer = LocalTransfer(),
                 decode_stall_timeout_s: float = 300.0, request_ttl_s: float = 600.0):
        self.llm, self.to_prefill, self.from_prefill, self.transfer = llm, to_prefill, from_prefill, transfer
        self.stall_timeout, self.ttl = decode_stall_timeout_s, request_ttl_s
        self._waiting: dict[str, tuple] = {}      # rid -> (ctx, sent_at)
        self._last_progress = time.monotonic()
        self.expired: list = []

    def add_request(self, prompt_ids, sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None) -> str:
        llm = self.llm
        llm._n += 1
        rid = request_id or f"di-{llm._n}"
        sp = sampling_params or SamplingParams()
        ctx = TextContext.from_prompt(prompt_ids, llm.max_length, rid, sp, llm.eos_token_ids)
        # reserve pages for the whole prompt now, so the transfer always has a place to land
        llm.kv.claim(ctx)
        llm.kv.alloc(ctx, extra_tokens=1)
        from ...entrypoints.llm import RequestRecord
        llm._records[rid] = RequestRecord(rid, ctx.tokens.prompt_len, arrival=ctx.arrival_time)
        self._waiting[rid] = (ctx, time.monotonic())
        self.to_prefill.put_nowait(PrefillRequest(rid, np.asarray(prompt_ids, dtype=np.int64), sp))
        return rid

    def _admit(self, res: PrefillResult) -> None:
        ctx, _ = self._waiting.pop(res.request_id)
        like = self.llm.kv.kv[: res.n_pages]
        pages = self.transfer.recv(like, res.pages)
        import_pages(self.llm.kv, res.request_id, pages)
        # the prompt is now "processed"; the first token becomes the active window of a decode request
        ctx.tokens.advance_processed()
        ctx.update(res.first_token)
        rec = self.llm._records[res.request_id]
        rec.first_token = rec.last_token = time.perf_counter()
        if ctx.is_done:
            rec.tokens.append(res.first_token)
            rec.finished = True
            self.llm.kv.release(res.request_id)
            self._finished_at_prefill.append(rec)
            return
        self.llm.scheduler._contexts[ctx.request_id] = ctx
        self.llm.scheduler.batch_constructor.enqueue_prefilled_request(ctx)

    _finished_at_prefill: list = []

    def step(self) -> list:
        now = time.monotonic()
        got = False
        while True:
            try:
                res = self.from_prefill.get_nowait()
            except queue.Empty:
                break
            if res.request_id in self._waiting:
                self._admit(res)
                got = True
        for rid, (ctx, sent) in list(self._waiting.items()):
            if now - sent > self.ttl:
                del self._waiting[rid]
                self.llm.kv.release(rid)
                self.llm._records.pop(rid, None)
                self.expired.append(rid)
        finished = list(self._finished_at_prefill)
        self._finished_at_prefill.clear()
        if self.llm.has_unfinished():
            finished += self.llm.step()
            got = True
        if got or not self._waiting:
            self._last_progress = now
        elif now - self._last_progress > self.stall_timeout:
            raise SystemExit(f"decode node stalled: no prefill result for {self.stall_timeout:.0f} s "
                             f"({len(self._waiting)} requests waiting)")
        return finished

    def has_unfinished(self) -> bool:
        return bool(self._waiting) or self.llm.has_unfinished() or bool(self._finished_at_prefill)
