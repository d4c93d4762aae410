"""Model worker: the process that owns the GPU and runs the scheduler loop.

Start-up: configure logging, run the pipeline factory (weights, KV cache, CUDA graphs), build
the scheduler on ZMQ queues, freeze the GC, signal readiness; then ``run_iteration`` forever,
beating a heartbeat every loop and backing off while idle. Reference:
max/python/max/serve/pipelines/model_worker.py:213 (factory :306, warm-up :351, scheduler :407,
gc freeze :472, loop :497-524), ``start_model_worker`` :579.
"""

from __future__ import annotations

import gc
import logging
import os
import time
import traceback
from typing import Callable, Optional

from .scheduler import SchedulerProgress, TokenGenerationScheduler, TokenGenerationSchedulerConfig
from .worker_interface import WorkerQueues, ZmqQueueSpec

logger = logging.getLogger("modular_b200.serve.model_worker")


class _SideChannel:
    """Small request/response RPC served once per loop (reset prefix cache, stats)."""

    def __init__(self, req_spec: ZmqQueueSpec, resp_spec: ZmqQueueSpec):
        self.req = req_spec.pull(bind=True)
        self.resp = resp_spec.push(bind=False)

    def service(self, handlers: dict) -> None:
        import queue

        while True:
            try:
                name, arg = self.req.get_nowait()
            except queue.Empty:
                return
            try:
                self.resp.put_nowait((name, True, handlers[name](arg)))
            except Exception as e:  # noqa: BLE001
                self.resp.put_nowait((name, False, repr(e)))


def scheduler_config_from(pipeline_config, llm) -> TokenGenerationSchedulerConfig:
    rt = pipeline_config.runtime
    return TokenGenerationSchedulerConfig(
        max_batch_size=llm.sched_config.max_batch_size if llm is not None else (rt.max_batch_size or 64),
        target_tokens_per_batch_ce=rt.max_batch_input_tokens,
        max_seq_len=llm.max_length if llm is not None else 1 << 20,
        enable_chunked_prefill=rt.enable_chunked_prefill,
        enable_in_flight_batching=rt.enable_in_flight_batching,
        kv_lookahead_tokens=1 if rt.enable_overlap_scheduler else 0)


def _drain(q, limit: int) -> list:
    """Everything waiting on a worker queue (at most ``limit`` items when limit > 0)."""
    import queue as _q

    out = []
    while limit <= 0 or len(out) < limit:
        try:
            out.append(q.get_nowait())
        except (_q.Empty, Exception):  # noqa: BLE001  (zmq queues raise their own Empty)
            break
    return out


class _PerRankFactory:
    """``factory(pipeline_config)``: the registry's build function with the pipeline config replaced (picklable,
    so that it can be handed to spawned ranks)."""

    def __init__(self, partial):
        self.func, self.args, self.kw = partial.func, partial.args, dict(partial.keywords or {})

    def __call__(self, pc):
        return self.func(pc, *self.args[1:], **self.kw)


def _rebind_factory(factory):
    return _PerRankFactory(factory)


def model_worker_main(factory: Callable, pipeline_config, queue_specs: dict, settings,
                      ready_event, alive_event, stop_event) -> None:
    """Entry point of the spawned process."""
    logging.basicConfig(level=getattr(logging, str(settings.log_level).upper(), logging.INFO),
                        format=f"%(asctime)s {settings.log_prefix or 'worker'} %(levelname)s %(name)s: %(message)s")
    try:
        t0 = time.perf_counter()
        # tensor parallelism: this process is rank 0; the other ranks are started here and fed in lock step
        tp_world = getattr(pipeline_config, "tensor_parallel_degree", 1) if pipeline_config is not None else 1
        ep_world = getattr(pipeline_config, "expert_parallel_degree", 1) if pipeline_config is not None else 1
        feed, followers, ep_feed = None, [], None
        if ep_world > 1 and getattr(factory, "func", None) is not None:
            # expert parallelism with data-parallel attention: this process is rank 0, it deals the requests to
            # the ranks and forwards everybody's outputs
            from . import tp_worker
            port = tp_worker.free_port()
            per_rank = _rebind_factory(factory)
            followers = tp_worker.start_followers(ep_world, port, per_rank, pipeline_config, settings,
                                                  main=tp_worker.ep_follower_main)
            pc0 = tp_worker.rank_config(pipeline_config, 0, ep_world)
            ctl = tp_worker.init_distributed(0, ep_world, port, pc0.model.device_ids[0])
            built = per_rank(pc0)
            ep_feed = tp_worker.ShardedFeed(ctl, 0, ep_world)
        elif tp_world > 1 and getattr(factory, "func", None) is not None:
            from . import tp_worker
            port = tp_worker.free_port()
            per_rank = _rebind_factory(factory)
            followers = tp_worker.start_followers(tp_world, port, per_rank, pipeline_config, settings)
            pc0 = tp_worker.rank_config(pipeline_config, 0, tp_world)
            ctl = tp_worker.init_distributed(0, tp_world, port, pc0.model.device_ids[0])
            built = per_rank(pc0)
            feed = tp_worker.LockstepFeed(ctl, 0)
        else:
            built = factory()
        llm = None
        if hasattr(built, "pipeline"):          # an LLM facade from the registry
            llm, pipeline, kv = built, built.pipeline, built.kv
        else:                                    # a bare pipeline (echo)
            pipeline, kv = built, getattr(built, "kv", None)
        queues = WorkerQueues(request=queue_specs["request"].pull(bind=True),
                              response=queue_specs["response"].push(bind=False),
                              cancel=queue_specs["cancel"].pull(bind=True))
        side = _SideChannel(queue_specs["rpc_req"], queue_specs["rpc_resp"])
        cfg = scheduler_config_from(pipeline_config, llm)
        # per-step metrics travel to the API process, which owns the Prometheus registry; a full queue drops them
        sink = None
        if "metrics" in queue_specs and str(getattr(settings.metric_recording, "value", settings.metric_recording)).upper() != "NOOP":
            mq = queue_specs["metrics"].push(bind=False)

            def sink(m):
                try:
                    mq.put_nowait(m.to_dict())
                except Exception:  # noqa: BLE001
                    pass
        ep_out = None
        if ep_feed is not None:
            import queue as _queue

            ep_out = _queue.SimpleQueue()      # this rank's outputs join the other ranks' in ep_feed.gather
            sched = TokenGenerationScheduler(cfg, pipeline, kv, ep_feed.requests, ep_out, ep_feed.cancels,
                                             metrics_sink=sink)
        elif feed is not None:
            # the scheduler reads the replicated stream; rank 0 alone answers the API process
            sched = TokenGenerationScheduler(cfg, pipeline, kv, feed.requests, queues.response, feed.cancels,
                                             metrics_sink=sink)
        else:
            sched = TokenGenerationScheduler(cfg, pipeline, kv, queues.request, queues.response, queues.cancel,
                                             metrics_sink=sink)
        def load_lora(arg):
            if llm is None:
                raise RuntimeError("this pipeline does not take LoRA adapters")
            from ..pipelines.lora import load_peft_adapter_files
            sd, alpha = load_peft_adapter_files(arg["path"])
            llm.load_lora(arg["name"], sd, alpha=arg.get("alpha") or alpha)
            return sorted(llm.pipeline.lora_manager.names())

        def unload_lora(arg):
            if llm is None or not llm.unload_lora(arg["name"]):
                raise RuntimeError(f"adapter {arg['name']!r} is not loaded")
            return sorted(llm.pipeline.lora_manager.names())

        def eplb_stats(arg):
            """Expert load per (MoE layer, expert) over all ranks, per-layer imbalance and the balancer's plan for
            the worst layer (reference: serve/pipelines/eplb_stats_rpc.py)."""
            from ..entrypoints.llm import merge_expert_load
            if ep_feed is None:
                raise RuntimeError("expert-load statistics need an expert-parallel engine (--ep-size)")
            stats = merge_expert_load(ep_feed.rank_loads, (arg or {}).get("slots_per_rank"))
            if stats is None:
                raise RuntimeError("no expert-load snapshot yet")
            return stats

        handlers = {
            "eplb_stats": eplb_stats,
            "load_lora": load_lora,
            "unload_lora": unload_lora,
            "list_loras": lambda _a: sorted(llm.pipeline.lora_manager.names())
            if llm is not None and llm.pipeline.lora_manager is not None else [],
            "reset_prefix_cache": lambda _a: bool(kv.reset_prefix_cache()) if kv is not None else False,
            "stats": lambda _a: {
                "steps": sched.total_steps, "pending": sched.batch_constructor.num_requests(),
                "kv_used_pct": kv.used_blocks_pct if kv is not None else 0.0,
                "cache_hit_rate": kv.cache_hit_rate if kv is not None else 0.0,
                "preemptions": sched.batch_constructor.total_preemptions},
        }
        from .telemetry import tracing

        tracing.configure_tracing(settings, service_name="modular_b200.model_worker")
        if tracing.batch_spans_enabled():
            # one span per scheduler iteration that ran a batch (kernel_trace_level >= 1)
            run_plain = sched.run_iteration

            def run_traced():
                with tracing.span("max.batch") as sp:
                    progress = run_plain()
                    m = sched.last_metrics
                    tracing.set_attributes(sp, **{"batch.type": m.batch_type, "batch.size": m.batch_size,
                                                  "batch.input_tokens": m.input_tokens,
                                                  "batch.output_tokens": m.output_tokens})
                return progress

            sched.run_iteration = run_traced
        # start-up objects go to the permanent generation (collections then only see what the loop allocates), free
        # allocator pages of the start-up peak go back to the system, and collections are timed from here on
        from .telemetry import gc_utils
        from .telemetry.metrics import METRICS

        frozen = gc_utils.freeze_startup_heap()
        gc_utils.trim_host_heap()
        gc_utils.install_gc_monitor(True, slow_ms=5.0 if settings.gc_debug else 50.0,
                                    top_types=settings.gc_debug_top_objects if settings.gc_debug else 0,
                                    observe=METRICS.gc_pause_ms.observe)
        logger.info("model worker ready in %.1f s (%d objects frozen)", time.perf_counter() - t0, frozen)
        ready_event.set()
        idle = 0
        while not stop_event.is_set():
            alive_event.set()
            if ep_feed is not None:
                from . import tp_worker
                if any(not p.is_alive() for p in followers):
                    raise RuntimeError("an expert-parallel rank died")
                _, responses, active = tp_worker.ep_iteration(
                    ep_feed, sched, llm.model, ep_out, _drain(queues.request, cfg.max_pending_requests),
                    _drain(queues.cancel, 0))
                for r in responses:
                    queues.response.put_nowait(r)
                side.service(handlers)
                if not active:
                    idle = min(idle + 1, 50)
                    time.sleep(min(0.0001 * (2 ** min(idle, 6)), 0.005))
                else:
                    idle = 0
                continue
            if feed is not None:
                if any(not p.is_alive() for p in followers):
                    raise RuntimeError("a tensor-parallel rank died")
                feed.exchange(_drain(queues.request, cfg.max_pending_requests), _drain(queues.cancel, 0))
            try:
                progress = sched.run_iteration()
            except Exception as e:      # noqa: BLE001
                # a single-process engine answers the requests it held with an error and goes on, as long as the
                # device still responds; ranks that step in lock-step cannot (the others are mid-step): they end
                if feed is not None or not hasattr(sched, "recover"):
                    raise
                logger.exception("a scheduler step failed; failing its requests and continuing")
                if not sched.recover(f"internal error in the model worker: {type(e).__name__}"):
                    raise
                progress = SchedulerProgress.MADE_PROGRESS
            side.service(handlers)
            if progress is SchedulerProgress.NO_PROGRESS:
                idle = min(idle + 1, 50)
                time.sleep(min(0.0001 * (2 ** min(idle, 6)), 0.005))
            else:
                idle = 0
        if feed is not None:
            feed.exchange(stop=True)
        if ep_feed is not None:
            ep_feed.exchange(stop=True)
    except BaseException:  # noqa: BLE001
        traceback.print_exc()
        os._exit(1)
