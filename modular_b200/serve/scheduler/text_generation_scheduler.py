"""Token-generation scheduler: the loop body of the model worker.

One ``run_iteration``: drain the request queue (bounded by ``max_pending_requests``),
construct a batch, execute it on the pipeline, move requests between queues, release
finished ones, push responses, service cancellations, record batch metrics.
Reference: max/python/max/serve/scheduler/text_generation_scheduler.py:86
(``run_iteration`` :197, ``_schedule`` :291).
"""

from __future__ import annotations

import enum
import queue
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

from ...pipelines.context import GenerationStatus, TextContext, TextGenerationOutput
from .batch_constructor import BatchType, SchedulerBatch, TextBatchConstructor
from .config import TokenGenerationSchedulerConfig


class SchedulerProgress(enum.Enum):
    MADE_PROGRESS = "made_progress"
    NO_PROGRESS = "no_progress"


@dataclass
class BatchMetrics:
    batch_type: str = "empty"
    batch_size: int = 0
    num_ce: int = 0
    num_tg: int = 0
    input_tokens: int = 0
    output_tokens: int = 0
    batch_time_s: float = 0.0
    kv_used_pct: float = 0.0
    cache_hit_rate: float = 0.0
    preemptions: int = 0
    pending_requests: int = 0
    batch_creation_s: float = 0.0
    context_tokens: int = 0          # resident context of the step's sequences (cached + new tokens)
    terminated: int = 0              # requests that finished in this step
    total_blocks: int = 0
    used_blocks: int = 0
    cache_hit_tokens: int = 0        # prompt tokens served from the prefix cache since the previous step
    cache_miss_tokens: int = 0
    used_host_kv_pct: float = 0.0
    used_disk_kv_pct: float = 0.0
    spec_steps: int = 0              # propose-and-verify passes of this step (one per request)
    spec_proposed: int = 0
    spec_accepted: int = 0
    spec_emitted: int = 0

    def to_dict(self) -> dict:
        """Flat form for the telemetry queue (keys as :func:`serve.telemetry.metrics.record_batch_metrics` reads them)."""
        import dataclasses
        d = dataclasses.asdict(self)
        d["used_kv_pct"] = d.pop("kv_used_pct")
        d["preempted"] = d.pop("preemptions")
        return d

    @property
    def prompt_throughput(self) -> float:
        return self.input_tokens / self.batch_time_s if self.batch_time_s > 0 else 0.0

    @property
    def generation_throughput(self) -> float:
        return self.output_tokens / self.batch_time_s if self.batch_time_s > 0 else 0.0


class TokenGenerationScheduler:
    def __init__(self, config: TokenGenerationSchedulerConfig, pipeline, kv=None,
                 request_queue=None, response_queue=None, cancel_queue=None,
                 metrics_sink: Optional[Callable[[BatchMetrics], None]] = None):
        self.config = config
        self.pipeline = pipeline
        self.kv = kv if kv is not None else getattr(pipeline, "kv", None)
        self.batch_constructor = TextBatchConstructor(config, self.kv, lambda: getattr(self.pipeline, "lora_manager", None))
        self.request_queue = request_queue if request_queue is not None else queue.SimpleQueue()
        self.response_queue = response_queue if response_queue is not None else queue.SimpleQueue()
        self.cancel_queue = cancel_queue if cancel_queue is not None else queue.SimpleQueue()
        self.metrics_sink = metrics_sink
        self.last_metrics = BatchMetrics()
        self._contexts: dict[str, TextContext] = {}
        self.total_steps = 0
        self._cache_seen = (0, 0)        # (hit tokens, queried tokens) already reported
        self._spec_seen = (0, 0, 0, 0)   # speculative-decoding counters already reported
        self._gate = None                # grammar compilations off the scheduler thread (created on first use)
        self._compiling: dict[str, TextContext] = {}
        # requests with task == "embed" are answered by an embeddings scheduler when the model can encode
        self.embeddings = None
        model = getattr(pipeline, "model", None)
        if model is not None and hasattr(model, "encode"):
            from .embeddings_scheduler import EmbeddingsScheduler
            own = getattr(model, "default_pooling", "last")    # what a request that names no pooling gets
            encode = lambda toks, pooling: model.encode(toks, own if pooling in (None, "default") else pooling)
            self.embeddings = EmbeddingsScheduler(encode, self.response_queue,
                                                  config.target_tokens_per_batch_ce, config.max_batch_size)

    # ------------------------------------------------------------ queue plumbing
    def _drain_requests(self) -> int:
        n, limit = 0, self.config.max_pending_requests
        model_generates = getattr(getattr(self.pipeline, "model", None), "generates", True)   # False: encoders
        while limit <= 0 or n < limit:
            try:
                ctx = self.request_queue.get_nowait()
            except queue.Empty:
                break
            except Exception:  # noqa: BLE001  (zmq queues raise their own Empty)
                break
            if getattr(ctx, "task", "generate") == "embed":
                if self.embeddings is None:
                    self.response_queue.put_nowait({ctx.request_id: TextGenerationOutput(
                        ctx.request_id, [], GenerationStatus.CANCELLED)})
                else:
                    self.embeddings.enqueue(ctx)
                n += 1
                continue
            if model_generates is False:
                self._fail(ctx, "this model serves embeddings (/v1/embeddings), not generation")
                n += 1
                continue
            if ctx.lora_name:
                # a request that names an adapter which is not (or no longer) loaded is refused here: it must
                # neither run on the base weights nor take the worker down
                mgr = getattr(self.pipeline, "lora_manager", None)
                if mgr is None or ctx.lora_name not in mgr.names():
                    self.response_queue.put_nowait({ctx.request_id: TextGenerationOutput(
                        ctx.request_id, [], GenerationStatus.CANCELLED)})
                    n += 1
                    continue
            self._contexts[ctx.request_id] = ctx
            if ctx.sampling_params.response_format is not None and ctx.grammar_state is None:
                # constrained request: its grammar is compiled off this thread and the request joins the prefill
                # queue when that is done; a grammar that does not compile fails this request only
                backend = getattr(self.pipeline, "structured", None)
                if backend is None:
                    self._fail(ctx, "this server was started without structured output (response_format)")
                    n += 1
                    continue
                if self._gate is None:
                    from ...pipelines.structured_output import GrammarGate

                    self._gate = GrammarGate(backend)
                self._gate.submit(ctx)
                self._compiling[ctx.request_id] = ctx
                n += 1
                continue
            self.batch_constructor.enqueue_new_request(ctx)
            n += 1
        return n

    def _fail(self, ctx: TextContext, message: str) -> None:
        self._contexts.pop(ctx.request_id, None)
        self.response_queue.put_nowait({ctx.request_id: TextGenerationOutput(
            ctx.request_id, [], GenerationStatus.ERROR, None, message)})

    def recover(self, message: str) -> bool:
        """After an exception inside a step: every request this scheduler knows fails with ``message``, pages and
        queues are released and the in-flight step is forgotten, so the worker can serve what comes next. False
        when the device no longer answers (the caller should then let the process end)."""
        for rid, ctx in list(self._contexts.items()):
            try:
                self.batch_constructor.release_request(rid, ctx)
            except Exception:      # noqa: BLE001 - the bookkeeping of a broken step may be half done
                pass
            self._fail(ctx, message)
        self._contexts.clear()
        if self._gate is not None:
            for rid in list(self._compiling):
                self._gate.release(rid)
        self._compiling.clear()
        bc = self.batch_constructor
        bc.ce_reqs.clear(), bc.tg_reqs.clear(), bc.draining.clear()
        if hasattr(self.pipeline, "abort_pending"):
            self.pipeline.abort_pending()
        try:
            import torch

            if torch.cuda.is_available() and getattr(self.pipeline, "on_gpu", False):
                torch.cuda.synchronize()
        except Exception:          # noqa: BLE001 - a sticky device error: nothing can run in this process any more
            return False
        return True

    def _admit_compiled(self) -> None:
        """Requests whose grammar compilation has finished: into the prefill queue, or failed with the reason."""
        for rid in [r for r, c in self._compiling.items() if self._gate.ready(c)]:
            ctx = self._compiling.pop(rid)
            if rid not in self._contexts:       # cancelled meanwhile
                self._gate.release(rid)
                continue
            err = self._gate.install(ctx)
            if err is not None:
                self._fail(ctx, err)
            else:
                self.batch_constructor.enqueue_new_request(ctx)

    def _handle_cancels(self) -> None:
        while True:
            try:
                rid = self.cancel_queue.get_nowait()
            except Exception:  # noqa: BLE001
                break
            ctx = self._contexts.pop(rid, None)
            if ctx is None:
                if self.embeddings is not None:
                    self.embeddings.cancel(rid)
                continue
            ctx.status = GenerationStatus.CANCELLED
            if self._compiling.pop(rid, None) is not None and self._gate is not None:
                self._gate.release(rid)
            self.batch_constructor.release_request(rid)
            self.response_queue.put_nowait({rid: TextGenerationOutput(rid, [], GenerationStatus.CANCELLED)})

    def add_request(self, ctx: TextContext) -> None:
        self.request_queue.put_nowait(ctx)

    def has_work(self) -> bool:
        return (self.batch_constructor.num_requests() > 0 or bool(self.batch_constructor.draining)
                or bool(self._compiling) or self.pipeline.has_pending() or bool(self.embeddings is not None and self.embeddings.pending))

    # ------------------------------------------------------------ one iteration
    def _finish(self, outputs: dict) -> None:
        done = [rid for rid, o in outputs.items() if o.is_done]
        for rid in done:
            if rid in self._contexts:
                self.batch_constructor.release_request(rid, self._contexts[rid])
                del self._contexts[rid]
        # outputs for requests already gone (cancelled, or extra speculative step) are dropped
        live = {rid: o for rid, o in outputs.items() if o.tokens or o.is_done}
        if live:
            self.response_queue.put_nowait(live)

    def run_iteration(self) -> SchedulerProgress:
        self._drain_requests()
        if self._compiling:
            self._admit_compiled()
        t0 = time.perf_counter()
        embedded = self.embeddings.run_iteration() if self.embeddings is not None else 0
        batch = self.batch_constructor.construct_batch()
        t_built = time.perf_counter()
        if not batch.contexts and not self.pipeline.has_pending():
            self._handle_cancels()
            return SchedulerProgress.MADE_PROGRESS if embedded else SchedulerProgress.NO_PROGRESS
        outputs = self.pipeline.execute(batch.contexts)
        self.batch_constructor.advance_requests(batch)
        self.total_steps += 1
        outputs = {rid: o for rid, o in outputs.items() if rid in self._contexts}
        self._finish(outputs)
        self._handle_cancels()
        dt = time.perf_counter() - t0
        kv = self.kv
        m = BatchMetrics(batch.batch_type.value, len(batch), batch.num_ce, batch.num_tg,
                         batch.input_tokens, sum(len(o.tokens) for o in outputs.values()), dt,
                         kv.used_blocks_pct if kv is not None else 0.0,
                         kv.cache_hit_rate if kv is not None else 0.0,
                         batch.preempted, self.batch_constructor.num_requests(),
                         batch_creation_s=t_built - t0,
                         context_tokens=sum(c.tokens.processed for c in batch.contexts),
                         terminated=sum(1 for o in outputs.values() if o.is_done))
        if kv is not None:
            hit, asked = kv.prefix_hit_tokens, kv.prefix_query_tokens
            m.cache_hit_tokens = hit - self._cache_seen[0]
            m.cache_miss_tokens = (asked - self._cache_seen[1]) - m.cache_hit_tokens
            self._cache_seen = (hit, asked)
            m.total_blocks, m.used_blocks = kv.pool.usable_blocks, kv.pool.used_blocks
            tiers = getattr(kv, "tiers", None)
            if tiers is not None:
                m.used_host_kv_pct = getattr(tiers, "host_used_pct", 0.0)
                m.used_disk_kv_pct = getattr(tiers, "disk_used_pct", 0.0)
        ss = getattr(self.pipeline, "spec_stats", None)
        if ss is not None:
            now = (ss.steps, ss.proposed, ss.accepted, ss.emitted)
            m.spec_steps, m.spec_proposed, m.spec_accepted, m.spec_emitted = (a - b for a, b in zip(now, self._spec_seen))
            self._spec_seen = now
        self.last_metrics = m
        if self.metrics_sink is not None:
            self.metrics_sink(m)
        return SchedulerProgress.MADE_PROGRESS
