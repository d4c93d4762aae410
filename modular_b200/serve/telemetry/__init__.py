"""Metrics, logging and tracing for the serving stack."""
