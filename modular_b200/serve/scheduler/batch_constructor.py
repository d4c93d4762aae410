"""Continuous-batching policy.

Requests live in two ordered queues: ``ce_reqs`` (context encoding: new prompts, prompts in
the middle of chunked prefill, and preempted requests that must re-encode) and ``tg_reqs``
(token generation: one new token per step). ``construct_batch`` builds the next step:

* **priority** - context encoding goes first unless in-flight batching is on (then every
  step carries all TG requests and fills the remaining token budget with CE chunks) or the
  KV cache is more than ``tg_priority_kv_percentage`` full (then decode drains first so
  pages free up);
* **chunked prefill** - the last CE context that does not fit the step's token budget has
  its active window shrunk to what fits, the rest runs in later steps;
* **KV pages** - every scheduled context gets pages through ``kv.alloc``; when the pool runs
  dry the *newest* TG request is preempted (pages released, context reset, moved to the
  front of the CE queue), and a CE request that cannot get pages simply waits.

Reference: max/python/max/serve/scheduler/batch_constructor/text_batch_constructor.py:263
(policy docstring :264-455, ``_identify_priority`` :965, ``_add_ce_requests`` :1057,
``_add_tg_requests`` :1161, ``construct_batch`` :1530).
"""

from __future__ import annotations

import enum
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

from ...kv_cache import InsufficientBlocksError, PagedKVCacheManager
from ...pipelines.context import TextContext
from .config import TokenGenerationSchedulerConfig
from .token_budget import ActiveTokenBudget, BudgetStatus, TotalContextTokenBudget


class BatchType(enum.Enum):
    CE = "context_encoding"
    TG = "token_generation"
    MIXED = "mixed"
    EMPTY = "empty"


@dataclass
class SchedulerBatch:
    contexts: list = field(default_factory=list)
    batch_type: BatchType = BatchType.EMPTY
    num_ce: int = 0
    num_tg: int = 0
    input_tokens: int = 0
    preempted: int = 0

    def __len__(self) -> int:
        return len(self.contexts)


class TextBatchConstructor:
    def __init__(self, config: TokenGenerationSchedulerConfig, kv: Optional[PagedKVCacheManager],
                 lora_manager=None):
        self.config = config
        self.kv = kv
        # a callable returning the pipeline's LoRA manager (it may be created after the scheduler), or None
        self.lora_manager = lora_manager
        self.ce_reqs: "OrderedDict[str, TextContext]" = OrderedDict()
        self.tg_reqs: "OrderedDict[str, TextContext]" = OrderedDict()
        self.draining: dict[str, TextContext] = {}   # finished, last token still in flight
        self.total_preemptions = 0

    def _kv_salt(self, ctx: TextContext) -> int:
        """Salt of the request's page hashes: the caller's ``cache_salt`` combined with the identity of the
        adapter the request runs on (reference: block_manager.py:134 passes ``ctx.cache_salt``)."""
        salt = int(ctx.cache_salt)
        if ctx.lora_name:
            mgr = self.lora_manager() if callable(self.lora_manager) else self.lora_manager
            if mgr is None:
                raise KeyError(f"request {ctx.request_id} names LoRA adapter {ctx.lora_name!r} but none is loaded")
            salt ^= mgr.cache_salt(ctx.lora_name)
        return salt & 0x7FFFFFFFFFFFFFFF

    # ------------------------------------------------------------ queue management
    def enqueue_new_request(self, ctx: TextContext) -> None:
        if ctx.request_id in self.ce_reqs or ctx.request_id in self.tg_reqs:
            raise ValueError(f"duplicate request id {ctx.request_id}")
        self.ce_reqs[ctx.request_id] = ctx

    def num_requests(self) -> int:
        return len(self.ce_reqs) + len(self.tg_reqs)

    def all_contexts(self):
        yield from self.ce_reqs.values()
        yield from self.tg_reqs.values()

    def contains(self, request_id: str) -> bool:
        return (request_id in self.ce_reqs or request_id in self.tg_reqs
                or request_id in self.draining)

    # optional hook ``on_release(request_id, n_tokens_with_kv)`` called just before a request's pages
    # are freed (a prefill-only engine exports them to the decode engine there)
    on_release = None

    def release_request(self, request_id: str, ctx: Optional[TextContext] = None) -> None:
        ctx = self.ce_reqs.pop(request_id, None) or self.tg_reqs.pop(request_id, None) or ctx
        ctx = self.draining.pop(request_id, None) or ctx
        self.ce_reqs.pop(request_id, None)
        self.tg_reqs.pop(request_id, None)
        if self.kv is not None:
            if self.on_release is not None and ctx is not None and self.kv.contains(request_id):
                self.on_release(request_id, ctx.tokens.processed)
            self.kv.release(request_id)

    def enqueue_prefilled_request(self, ctx: TextContext) -> None:
        """A request whose prompt KV is already in this engine's cache (disaggregated decode): it joins
        the token-generation queue directly. Its pages must have been claimed and filled."""
        if ctx.request_id in self.ce_reqs or ctx.request_id in self.tg_reqs:
            raise ValueError(f"duplicate request id {ctx.request_id}")
        self.tg_reqs[ctx.request_id] = ctx

    # ------------------------------------------------------------ policy pieces
    def _identify_priority(self) -> BatchType:
        cfg = self.config
        if not self.ce_reqs:
            return BatchType.TG
        if not self.tg_reqs:
            return BatchType.CE
        if self.kv is not None and self.kv.used_blocks_pct > cfg.tg_priority_kv_percentage:
            return BatchType.TG
        if cfg.batch_strategy == "decode_first":
            return BatchType.TG
        return BatchType.CE

    def _preempt_newest_tg(self, exclude: set) -> bool:
        for rid in reversed(list(self.tg_reqs.keys())):
            if rid in exclude:
                continue
            ctx = self.tg_reqs.pop(rid)
            if ctx.pending_future:
                # its last token is still on the device; re-encoding needs the value
                self.tg_reqs[rid] = ctx
                self.tg_reqs.move_to_end(rid, last=False)
                continue
            if self.kv is not None:
                self.kv.release(rid)
            ctx.reset()
            self.ce_reqs[rid] = ctx
            self.ce_reqs.move_to_end(rid, last=False)
            self.total_preemptions += 1
            if self.kv is not None:
                self.kv.preemptions += 1
            return True
        return False

    def _add_tg_requests(self, batch: SchedulerBatch, budget: ActiveTokenBudget) -> None:
        cfg = self.config
        scheduled: set = set()
        for rid in list(self.tg_reqs.keys()):
            if rid not in self.tg_reqs:      # preempted while we iterated
                continue
            if len(batch) >= cfg.max_batch_size or budget.remaining <= 0:
                break
            ctx = self.tg_reqs[rid]
            if self.kv is not None:
                while True:
                    try:
                        self.kv.alloc(ctx, cfg.kv_lookahead_tokens)
                        break
                    except InsufficientBlocksError:
                        batch.preempted += 1
                        if not self._preempt_newest_tg(scheduled | {rid}):
                            # nothing else to evict: preempt this one and stop
                            if not ctx.pending_future:
                                self.tg_reqs.pop(rid)
                                self.kv.release(rid)
                                ctx.reset()
                                self.ce_reqs[rid] = ctx
                                self.ce_reqs.move_to_end(rid, last=False)
                                self.total_preemptions += 1
                            ctx = None
                            break
                if ctx is None:
                    break
            budget.used += ctx.tokens.active_length
            batch.contexts.append(ctx)
            batch.num_tg += 1
            scheduled.add(rid)

    def _add_ce_requests(self, batch: SchedulerBatch, budget: ActiveTokenBudget,
                         total: TotalContextTokenBudget) -> None:
        cfg = self.config
        for rid in list(self.ce_reqs.keys()):
            if len(batch) >= cfg.max_batch_size or budget.remaining <= 0:
                break
            ctx = self.ce_reqs[rid]
            if ctx.pending_future:
                continue
            if self.kv is not None:
                if not self.kv.contains(rid):
                    # also the path of a re-claim after preemption: the salt is recomputed from the request
                    self.kv.claim(ctx, salt=self._kv_salt(ctx))
                # prefix-cache lookup on the whole prompt first: it moves the window start
                self.kv.lookup_prefix(ctx)
            st = budget.status_after_context(ctx)       # may chunk the window
            if st is BudgetStatus.BUDGET_EXHAUSTED:
                break
            n_active = ctx.tokens.active_length
            ok = total.status_after_context(ctx) is not BudgetStatus.BUDGET_EXHAUSTED
            if ok and self.kv is not None:
                try:
                    self.kv.alloc(ctx)
                except InsufficientBlocksError:
                    ok = False
            if not ok:
                # leave the request queued with its full window; it retries next step
                budget.used -= n_active
                ctx.tokens.active_end = len(ctx.tokens)
                break
            batch.contexts.append(ctx)
            batch.num_ce += 1
            if st is BudgetStatus.BUDGET_REACHED:
                break

    # ------------------------------------------------------------ entry points
    def construct_batch(self) -> SchedulerBatch:
        cfg = self.config
        batch = SchedulerBatch()
        budget = ActiveTokenBudget(cfg.target_tokens_per_batch_ce, cfg.enable_chunked_prefill,
                                   cfg.chunked_prefill_min_chunk_size, cfg.step_token_alignment)
        total = TotalContextTokenBudget(cfg.max_batch_total_tokens,
                                        self.kv.page_size if self.kv is not None else 1)
        if cfg.enable_in_flight_batching:
            self._add_tg_requests(batch, budget)
            self._add_ce_requests(batch, budget, total)
        else:
            prio = self._identify_priority()
            if prio is BatchType.CE:
                self._add_ce_requests(batch, budget, total)
                if not batch.contexts:
                    self._add_tg_requests(batch, budget)
            else:
                self._add_tg_requests(batch, budget)
                if not batch.contexts:
                    self._add_ce_requests(batch, budget, total)
        batch.input_tokens = sum(c.tokens.active_length for c in batch.contexts)
        if batch.num_ce and batch.num_tg:
            batch.batch_type = BatchType.MIXED
        elif batch.num_ce:
            batch.batch_type = BatchType.CE
        elif batch.num_tg:
            batch.batch_type = BatchType.TG
        return batch

    def advance_requests(self, batch: SchedulerBatch) -> None:
        """After the pipeline consumed the batch: move contexts between queues."""
        for ctx in batch.contexts:
            rid = ctx.request_id
            if ctx.is_done:
                self.ce_reqs.pop(rid, None)
                self.tg_reqs.pop(rid, None)
                if ctx.pending_future:
                    self.draining[rid] = ctx
                continue
            if ctx.needs_ce:
                # more prompt chunks to go
                if rid not in self.ce_reqs:
                    self.tg_reqs.pop(rid, None)
                    self.ce_reqs[rid] = ctx
                    self.ce_reqs.move_to_end(rid, last=False)
            else:
                if rid in self.ce_reqs:
                    del self.ce_reqs[rid]
                if rid not in self.tg_reqs:
                    self.tg_reqs[rid] = ctx
