"""Scheduler configuration (reference: max/python/max/serve/scheduler/config.py:20)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class TokenGenerationSchedulerConfig:
    max_batch_size: int = 256                  # sequences per step (TG + CE)
    target_tokens_per_batch_ce: int = 8192     # new-token budget of one step (max_batch_input_tokens)
    max_seq_len: int = 131072
    max_batch_total_tokens: int = 0            # cap on resident context tokens (0 = unlimited)
    enable_chunked_prefill: bool = True
    chunked_prefill_min_chunk_size: int = 16
    step_token_alignment: int = 0              # trim prompt chunks so steps land on multiples of this (0 = off)
    enable_in_flight_batching: bool = False    # mix CE chunks into TG steps
    max_pending_requests: int = 0              # requests drained from the queue per iteration (0 = all)
    tg_priority_kv_percentage: float = 0.90    # above this KV usage decode goes first
    data_parallel_degree: int = 1
    num_speculative_tokens: int = 0
    batch_strategy: str = "prefill_first"      # prefill_first | decode_first | balanced
    kv_lookahead_tokens: int = 1               # pages reserved ahead for in-flight future tokens

    def __post_init__(self):
        if self.max_batch_size < 1:
            raise ValueError("max_batch_size must be >= 1")
        if self.target_tokens_per_batch_ce < 1:
            raise ValueError("target_tokens_per_batch_ce must be >= 1")
        if self.batch_strategy not in ("prefill_first", "decode_first", "balanced"):
            raise ValueError(f"unknown batch strategy {self.batch_strategy!r}")
