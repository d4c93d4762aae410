"""HTTP routers (OpenAI-compatible first; KServe / SageMaker thin adapters)."""
