"""Serving metrics with the reference's ``maxserve.*`` names, exported for Prometheus.

Reference: max/python/max/serve/telemetry/metrics.py (instruments :86-630). Recording goes
through a process-global ``METRICS`` object; ``configure_metrics(NOOP)`` swaps every
instrument for a no-op so the hot path pays nothing when metrics are off.
"""

from __future__ import annotations

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest

_MS_BUCKETS = (1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000, 60000)


class _Noop:
    def inc(self, *_a, **_k): pass
    def observe(self, *_a, **_k): pass
    def set(self, *_a, **_k): pass


class Metrics:
    def __init__(self, enabled: bool = True):
        self.registry = CollectorRegistry()
        self.enabled = enabled
        mk_c = (lambda n, d: Counter(n, d, registry=self.registry)) if enabled else (lambda n, d: _Noop())
        mk_h = (lambda n, d: Histogram(n, d, buckets=_MS_BUCKETS, registry=self.registry)) if enabled else (lambda n, d: _Noop())
        mk_g = (lambda n, d: Gauge(n, d, registry=self.registry)) if enabled else (lambda n, d: _Noop())
        self.request_count = mk_c("maxserve_request_count", "requests received")
        self.request_errors = mk_c("maxserve_request_errors", "requests that ended with an error")
        self.input_tokens = mk_c("maxserve_num_input_tokens", "prompt tokens received")
        self.output_tokens = mk_c("maxserve_num_output_tokens", "tokens generated")
        self.request_time_ms = mk_h("maxserve_request_time_ms", "end-to-end request latency")
        self.ttft_ms = mk_h("maxserve_time_to_first_token_ms", "time to first token")
        self.itl_ms = mk_h("maxserve_itl_ms", "inter-token latency")
        self.tpot_ms = mk_h("maxserve_time_per_output_token_ms", "time per output token")
        self.queue_depth = mk_g("maxserve_num_requests_queued", "requests waiting for the worker")
        self.running = mk_g("maxserve_num_requests_running", "requests in flight")
        self.batch_size = mk_h("maxserve_batch_size", "sequences per scheduler step")
        self.batch_time_ms = mk_h("maxserve_batch_execution_time_ms", "scheduler step time")
        self.cache_hit_rate = mk_g("maxserve_cache_hit_rate", "prefix cache hit rate")
        self.cache_used_pct = mk_g("maxserve_cache_used_blocks_pct", "KV pages in use")
        self.preemptions = mk_c("maxserve_cache_preemption_count", "requests preempted")

    def render(self) -> bytes:
        return generate_latest(self.registry)


METRICS = Metrics(True)


def configure_metrics(method: str) -> Metrics:
    """``NOOP`` disables recording; every other method records in-process."""
    global METRICS
    new = Metrics(str(method).upper() != "NOOP")
    METRICS.__dict__.update(new.__dict__)
    return METRICS
