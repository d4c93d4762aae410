"""Serving metrics with the reference's ``maxserve.*`` names, exported for Prometheus.

Reference: max/python/max/serve/telemetry/metrics.py (instruments :86-630, metric clients :830). Prometheus
spells the dots as underscores (``maxserve.cache.hits`` -> ``maxserve_cache_hits``). Recording goes through a
process-global ``METRICS`` object; ``configure_metrics(NOOP)`` swaps every instrument for a no-op so the hot
path pays nothing when metrics are off.

The request-level instruments are recorded in the API process. The batch- and cache-level ones are produced by
the scheduler inside the model worker: it pushes one ``BatchMetrics`` per step onto a telemetry queue and the API
process replays them into the instruments with :func:`record_batch_metrics` (the role of the reference's process
metric client, ``telemetry/process_controller.py:135``).
"""

from __future__ import annotations

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest

_MS_BUCKETS = (1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000, 60000)
_COUNT_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 65536)
_RATE_BUCKETS = (10, 100, 1000, 3000, 10000, 30000, 100000, 300000, 1000000)
_FRAC_BUCKETS = (0.0, 0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0)


class _Noop:
    def inc(self, *_a, **_k): pass
    def observe(self, *_a, **_k): pass
    def set(self, *_a, **_k): pass


class Metrics:
    def __init__(self, enabled: bool = True):
        self.registry = CollectorRegistry()
        self.enabled = enabled
        reg = self.registry
        mk_c = (lambda n, d: Counter(n, d, registry=reg)) if enabled else (lambda n, d: _Noop())
        mk_g = (lambda n, d: Gauge(n, d, registry=reg)) if enabled else (lambda n, d: _Noop())

        def mk_h(n, d, buckets=_MS_BUCKETS):
            return Histogram(n, d, buckets=buckets, registry=reg) if enabled else _Noop()

        # ---- requests (API process)
        self.request_count = mk_c("maxserve_request_count", "requests received")
        self.request_errors = mk_c("maxserve_request_errors", "requests that ended with an error")
        self.input_tokens = mk_c("maxserve_num_input_tokens", "prompt tokens received")
        self.input_characters = mk_c("maxserve_num_input_characters", "prompt characters received")
        self.output_tokens = mk_c("maxserve_num_output_tokens", "tokens generated")
        self.input_tokens_per_request = mk_h("maxserve_input_tokens_per_request", "prompt tokens of a request", _COUNT_BUCKETS)
        self.output_tokens_per_request = mk_h("maxserve_output_tokens_per_request", "generated tokens of a request", _COUNT_BUCKETS)
        self.request_time_ms = mk_h("maxserve_request_time_ms", "end-to-end request latency")
        self.ttft_ms = mk_h("maxserve_time_to_first_token_ms", "time to first token")
        self.itl_ms = mk_h("maxserve_itl_ms", "inter-token latency")
        self.tpot_ms = mk_h("maxserve_time_per_output_token_ms", "time per output token")
        self.input_processing_ms = mk_h("maxserve_input_processing_time_ms", "tokenisation and request set-up")
        self.output_processing_ms = mk_h("maxserve_output_processing_time_ms", "detokenisation of one chunk")
        self.queue_depth = mk_g("maxserve_num_requests_queued", "requests waiting for the worker")
        self.running = mk_g("maxserve_num_requests_running", "requests in flight")
        self.tool_call_errors = mk_c("maxserve_tool_call_conformance_errors", "answers whose tool-call JSON did not parse")
        self.response_format_errors = mk_c("maxserve_response_format_conformance_errors",
                                           "constrained answers that do not parse as their format")
        self.model_load_time_ms = mk_g("maxserve_model_load_time_ms", "time the model worker took to become ready")
        self.pipeline_load = mk_c("maxserve_pipeline_load", "pipelines loaded")
        # ---- scheduler steps (model worker, replayed here)
        self.batch_size = mk_h("maxserve_batch_size", "sequences per scheduler step", _COUNT_BUCKETS)
        self.batch_time_ms = mk_h("maxserve_batch_execution_time_ms", "scheduler step time")
        self.batch_creation_ms = mk_h("maxserve_batch_creation_time_ms", "time to build a batch")
        self.batch_input_tokens = mk_h("maxserve_batch_input_tokens", "tokens fed to a step", _COUNT_BUCKETS)
        self.batch_context_tokens = mk_h("maxserve_batch_context_tokens", "resident context tokens of a step", _COUNT_BUCKETS)
        self.batch_prompt_tps = mk_h("maxserve_batch_prompt_throughput", "prompt tokens per second of a step", _RATE_BUCKETS)
        self.batch_generation_tps = mk_h("maxserve_batch_generation_throughput", "generated tokens per second of a step", _RATE_BUCKETS)
        self.batch_pending = mk_g("maxserve_batch_pending_reqs", "requests waiting in the scheduler")
        self.batch_terminated = mk_c("maxserve_batch_terminated_reqs", "requests that finished")
        # ---- KV cache
        self.cache_hit_rate = mk_g("maxserve_cache_hit_rate", "prefix cache hit rate")
        self.cache_used_pct = mk_g("maxserve_cache_used_kv_pct", "device KV pages in use (fraction)")
        self.cache_used_host_pct = mk_g("maxserve_cache_used_host_kv_pct", "host-tier KV pages in use (fraction)")
        self.cache_used_disk_pct = mk_g("maxserve_cache_used_disk_kv_pct", "disk-tier KV pages in use (fraction)")
        self.cache_total_blocks = mk_g("maxserve_cache_num_total_blocks", "device KV pages")
        self.cache_used_blocks = mk_g("maxserve_cache_num_used_blocks", "device KV pages in use")
        self.cache_hits = mk_c("maxserve_cache_hits", "prompt tokens served from the prefix cache")
        self.cache_misses = mk_c("maxserve_cache_misses", "prompt tokens that had to be computed")
        self.preemptions = mk_c("maxserve_cache_preemption_count", "requests preempted")
        self.prefix_coverage = mk_h("maxserve_cache_request_prefix_coverage", "fraction of a prompt found in the cache", _FRAC_BUCKETS)
        # ---- speculative decoding, structured output
        self.spec_acceptance_len = mk_h("maxserve_spec_decode_avg_acceptance_length", "tokens emitted per verification step",
                                        (1, 1.5, 2, 2.5, 3, 4, 5, 6, 8))
        self.spec_acceptance_rate = mk_g("maxserve_spec_decode_acceptance_rate", "accepted / proposed draft tokens")
        self.grammar_rejections = mk_c("maxserve_structured_output_grammar_rejections", "sampled tokens a grammar refused")
        self.gc_pause_ms = mk_h("maxserve_gc_pause_ms", "stop-the-world time of a Python garbage collection",
                                (0.1, 0.5, 1, 2, 5, 10, 20, 50, 100, 500))
        # ---- did generated tool calls / JSON answers match the declared schemas (observation only)
        self.tool_call_nonconforming = mk_c("maxserve_tool_call_nonconforming",
                                            "tool calls with unknown names, unparsable or schema-violating arguments")
        self.response_format_nonconforming = mk_c("maxserve_response_format_nonconforming",
                                                  "JSON answers that did not parse or did not match the requested schema")

    def render(self) -> bytes:
        return generate_latest(self.registry)


METRICS = Metrics(True)


def configure_metrics(method: str) -> Metrics:
    """``NOOP`` disables recording; every other method records in-process."""
    global METRICS
    new = Metrics(str(method).upper() != "NOOP")
    METRICS.__dict__.update(new.__dict__)
    return METRICS


def record_batch_metrics(m: dict) -> None:
    """Replays one scheduler step's metrics (a ``BatchMetrics`` as a dict, sent by the model worker)."""
    M = METRICS
    M.batch_size.observe(m.get("batch_size", 0))
    M.batch_time_ms.observe(m.get("batch_time_s", 0.0) * 1e3)
    M.batch_creation_ms.observe(m.get("batch_creation_s", 0.0) * 1e3)
    M.batch_input_tokens.observe(m.get("input_tokens", 0))
    M.batch_context_tokens.observe(m.get("context_tokens", 0))
    dt = m.get("batch_time_s", 0.0)
    if dt > 0:
        if m.get("num_ce", 0):
            M.batch_prompt_tps.observe(m.get("input_tokens", 0) / dt)
        if m.get("output_tokens", 0):
            M.batch_generation_tps.observe(m.get("output_tokens", 0) / dt)
    M.batch_pending.set(m.get("pending_requests", 0))
    M.batch_terminated.inc(m.get("terminated", 0))
    M.cache_hit_rate.set(m.get("cache_hit_rate", 0.0))
    M.cache_used_pct.set(m.get("used_kv_pct", 0.0))
    M.cache_used_host_pct.set(m.get("used_host_kv_pct", 0.0))
    M.cache_used_disk_pct.set(m.get("used_disk_kv_pct", 0.0))
    M.cache_total_blocks.set(m.get("total_blocks", 0))
    M.cache_used_blocks.set(m.get("used_blocks", 0))
    M.cache_hits.inc(m.get("cache_hit_tokens", 0))
    M.cache_misses.inc(m.get("cache_miss_tokens", 0))
    M.preemptions.inc(m.get("preempted", 0))
    for cov in m.get("prefix_coverage", ()):
        M.prefix_coverage.observe(cov)
    if m.get("spec_steps", 0):
        M.spec_acceptance_len.observe(m.get("spec_emitted", 0) / m["spec_steps"])
        if m.get("spec_proposed", 0):
            M.spec_acceptance_rate.set(m.get("spec_accepted", 0) / m["spec_proposed"])
