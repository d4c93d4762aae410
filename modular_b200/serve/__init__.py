"""Serving stack: OpenAI-compatible API server, worker transport, scheduler, telemetry."""
