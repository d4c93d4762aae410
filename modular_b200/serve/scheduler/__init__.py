"""Schedulers (reference: max/python/max/serve/scheduler/__init__.py:72 ``load_scheduler``)."""

from .batch_constructor import BatchType, SchedulerBatch, TextBatchConstructor
from .config import TokenGenerationSchedulerConfig
from .text_generation_scheduler import BatchMetrics, SchedulerProgress, TokenGenerationScheduler
from .token_budget import ActiveTokenBudget, BudgetStatus, TotalContextTokenBudget

__all__ = ["BatchType", "SchedulerBatch", "TextBatchConstructor", "TokenGenerationSchedulerConfig",
           "BatchMetrics", "SchedulerProgress", "TokenGenerationScheduler", "ActiveTokenBudget",
           "BudgetStatus", "TotalContextTokenBudget", "load_scheduler"]


def load_scheduler(pipeline, config: TokenGenerationSchedulerConfig, pipeline_role: str = "prefill_and_decode",
                   **queues):
    """Pick the scheduler for a pipeline and role."""
    if pipeline_role != "prefill_and_decode":
        raise NotImplementedError(
            f"pipeline_role={pipeline_role!r}: disaggregated prefill/decode scheduling is not built yet")
    return TokenGenerationScheduler(config, pipeline, **queues)
