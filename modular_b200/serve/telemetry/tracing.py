"""Request and batch tracing with OpenTelemetry.

``configure_tracing(settings)`` installs a tracer provider when telemetry is enabled and a destination is
configured: the standard ``OTEL_EXPORTER_OTLP_ENDPOINT`` / ``OTEL_EXPORTER_OTLP_TRACES_ENDPOINT`` variables
(OTLP over HTTP), or ``MAX_SERVE_TRACE_FILE`` (one JSON object per finished span). Without a destination, or with
``disable_telemetry``, every call here is a no-op; nothing is sent anywhere by default. The API process opens one
server span per HTTP request (continuing an incoming W3C ``traceparent``) with child spans for tokenisation and
generation; the model worker opens one ``max.batch`` span per scheduler iteration from ``kernel_trace_level`` 1 up.

Reference: max/python/max/serve/telemetry/common.py:644 (``configure_tracing``), :676 (``batch_spans_enabled``).
"""

from __future__ import annotations

import contextlib
import json
import os
import threading
from typing import Optional

_TRACER = None
_PROVIDER = None
_BATCH_SPANS = False
_LOCK = threading.Lock()


class _JsonFileExporter:
    """Span exporter that appends one JSON line per span (name, ids, times in ns, attributes)."""

    def __init__(self, path: str):
        self.path = path
        self._lock = threading.Lock()

    def export(self, spans):
        from opentelemetry.sdk.trace.export import SpanExportResult

        with self._lock, open(self.path, "a") as f:
            for s in spans:
                ctx = s.get_span_context()
                f.write(json.dumps({
                    "name": s.name, "trace_id": f"{ctx.trace_id:032x}", "span_id": f"{ctx.span_id:016x}",
                    "parent_id": f"{s.parent.span_id:016x}" if s.parent is not None else None,
                    "start_ns": s.start_time, "end_ns": s.end_time, "attributes": dict(s.attributes or {})}) + "\n")
        return SpanExportResult.SUCCESS

    def shutdown(self):
        pass

    def force_flush(self, timeout_millis: int = 30000):
        return True


def configure_tracing(settings, exporter=None, service_name: str = "modular_b200.serve") -> bool:
    """Install the tracer. ``exporter`` overrides the destination (tests pass an in-memory exporter).
    Returns whether tracing is on."""
    global _TRACER, _PROVIDER, _BATCH_SPANS
    with _LOCK:
        _BATCH_SPANS = int(getattr(settings, "kernel_trace_level", 0) or 0) >= 1
        if getattr(settings, "disable_telemetry", True) and exporter is None:
            _TRACER = None
            return False
        processor = None
        from opentelemetry.sdk.trace.export import BatchSpanProcessor, SimpleSpanProcessor

        if exporter is not None:
            processor = SimpleSpanProcessor(exporter)
        elif os.environ.get("OTEL_EXPORTER_OTLP_ENDPOINT") or os.environ.get("OTEL_EXPORTER_OTLP_TRACES_ENDPOINT"):
            from opentelemetry.exporter.otlp.proto.http.trace_exporter import OTLPSpanExporter

            processor = BatchSpanProcessor(OTLPSpanExporter())
        elif os.environ.get("MAX_SERVE_TRACE_FILE"):
            processor = SimpleSpanProcessor(_JsonFileExporter(os.environ["MAX_SERVE_TRACE_FILE"]))
        if processor is None:
            _TRACER = None
            return False
        from opentelemetry.sdk.resources import Resource
        from opentelemetry.sdk.trace import TracerProvider

        _PROVIDER = TracerProvider(resource=Resource.create({"service.name": service_name}))
        _PROVIDER.add_span_processor(processor)
        _TRACER = _PROVIDER.get_tracer("modular_b200.serve")
        return True


def tracing_enabled() -> bool:
    return _TRACER is not None


def batch_spans_enabled() -> bool:
    return _TRACER is not None and _BATCH_SPANS


def shutdown_tracing() -> None:
    global _TRACER, _PROVIDER
    with _LOCK:
        if _PROVIDER is not None:
            _PROVIDER.shutdown()
        _TRACER = _PROVIDER = None


@contextlib.contextmanager
def span(name: str, attributes: Optional[dict] = None, traceparent: Optional[str] = None, kind: str = "internal"):
    """A span as a context manager; yields the span (or None when tracing is off). ``traceparent``: the W3C header
    of an incoming request, whose trace this span continues."""
    if _TRACER is None:
        yield None
        return
    from opentelemetry import trace
    from opentelemetry.trace.propagation.tracecontext import TraceContextTextMapPropagator

    ctx = TraceContextTextMapPropagator().extract({"traceparent": traceparent}) if traceparent else None
    k = trace.SpanKind.SERVER if kind == "server" else trace.SpanKind.INTERNAL
    with _TRACER.start_as_current_span(name, context=ctx, kind=k, attributes=attributes or {}) as s:
        yield s


def current_traceparent() -> Optional[str]:
    """The ``traceparent`` value of the current span (handed to outgoing responses and to the worker)."""
    if _TRACER is None:
        return None
    from opentelemetry.trace.propagation.tracecontext import TraceContextTextMapPropagator

    carrier: dict = {}
    TraceContextTextMapPropagator().inject(carrier)
    return carrier.get("traceparent")


def set_attributes(s, **attrs) -> None:
    if s is not None:
        for k, v in attrs.items():
            if v is not None:
                s.set_attribute(k, v)
