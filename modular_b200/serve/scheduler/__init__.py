"""Schedulers (reference: max/python/max/serve/scheduler/__init__.py:72 ``load_scheduler``)."""

from .batch_constructor import BatchType, SchedulerBatch, TextBatchConstructor
from .config import TokenGenerationSchedulerConfig
from .dp_padding import DPBatchPadder, DPPaddingInfo
from .one_shot_scheduler import OneShotScheduler
from .text_generation_scheduler import BatchMetrics, SchedulerProgress, TokenGenerationScheduler
from .token_budget import ActiveTokenBudget, BudgetStatus, TotalContextTokenBudget

__all__ = ["BatchType", "SchedulerBatch", "TextBatchConstructor", "TokenGenerationSchedulerConfig",
           "BatchMetrics", "SchedulerProgress", "TokenGenerationScheduler", "ActiveTokenBudget",
           "BudgetStatus", "TotalContextTokenBudget", "load_scheduler", "DPBatchPadder", "DPPaddingInfo",
           "OneShotScheduler"]


def load_scheduler(pipeline, config: TokenGenerationSchedulerConfig, pipeline_role: str = "prefill_and_decode",
                   **queues):
    """Pick the scheduler for a pipeline and role. ``prefill_only`` / ``decode_only`` engines are driven by
    :class:`disaggregated.PrefillNode` / :class:`disaggregated.DecodeNode`, which wrap an engine built with
    the ordinary scheduler (the role changes who feeds it and where finished prefills go)."""
    if pipeline_role not in ("prefill_and_decode", "prefill_only", "decode_only"):
        raise ValueError(f"unknown pipeline_role {pipeline_role!r}")
    if getattr(pipeline, "one_shot", False):
        # pipelines whose every request finishes in one call (reference: scheduler/__init__.py:72-171 picks the
        # scheduler by pipeline class)
        return OneShotScheduler(pipeline, queues.get("request_queue"), queues.get("response_queue"),
                                queues.get("cancel_queue"), config.max_batch_size, config.target_tokens_per_batch_ce)
    return TokenGenerationScheduler(config, pipeline, **queues)
