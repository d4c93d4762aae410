"""Token budgets that bound one scheduler step.

``ActiveTokenBudget`` caps the number of *new* tokens a step processes and, when chunked
prefill is enabled, shrinks the last context's active window so the step lands exactly on
the cap. ``TotalContextTokenBudget`` caps the page-aligned resident context of the batch.
Reference: max/python/max/serve/scheduler/batch_constructor/token_budget.py:224, :346.
"""

from __future__ import annotations

import enum


class BudgetStatus(enum.Enum):
    BUDGET_AVAILABLE = 0   # context added, room remains
    BUDGET_REACHED = 1     # context added (possibly chunked), the step is full
    BUDGET_EXHAUSTED = 2   # context not added


class ActiveTokenBudget:
    """``align`` > 0 makes steps land on whole multiples of ``align`` tokens when they would otherwise
    overshoot one by less than ``align // 4``: a prompt chunk that would bring a step to 1088 tokens is cut
    so the step has 1024 and the 64 left over ride along with the next step. The GEMMs tile tokens in
    blocks of up to 256 and weight rows in blocks of 128; with 32 weight-row blocks (N = 4096) a step of
    1024 tokens is 128 CTAs - one wave on 148 SMs - while 1088 tokens need 160 CTAs and a second, almost
    empty wave that nearly doubles the time of those GEMMs."""

    def __init__(self, capacity: int, allow_chunking: bool = True, min_chunk: int = 1, align: int = 0):
        self.capacity = capacity
        self.used = 0
        self.allow_chunking = allow_chunking
        self.min_chunk = max(1, min_chunk)
        self.align = max(0, align)

    @property
    def remaining(self) -> int:
        return self.capacity - self.used

    def status_after_context(self, ctx) -> BudgetStatus:
        """Try to add ``ctx``; may chunk its active window. Mutates ``used`` on success."""
        n = ctx.tokens.active_length
        rem = self.remaining
        if rem <= 0:
            return BudgetStatus.BUDGET_EXHAUSTED
        if n <= rem:
            if self.align and self.allow_chunking:
                total = self.used + n
                over = total % self.align
                keep = n - over                      # lands the step on a multiple of `align`
                if total > self.align and 0 < over < self.align // 4 and keep >= self.min_chunk:
                    ctx.tokens.chunk(keep)
                    self.used += ctx.tokens.active_length
                    return BudgetStatus.BUDGET_REACHED
            self.used += n
            return BudgetStatus.BUDGET_REACHED if self.used == self.capacity else BudgetStatus.BUDGET_AVAILABLE
        if not self.allow_chunking or rem < min(self.min_chunk, n):
            return BudgetStatus.BUDGET_EXHAUSTED
        ctx.tokens.chunk(rem)
        self.used += ctx.tokens.active_length
        return BudgetStatus.BUDGET_REACHED


class TotalContextTokenBudget:
    def __init__(self, capacity: int, page_size: int):
        self.capacity = capacity
        self.page_size = page_size
        self.used = 0

    def _aligned(self, n: int) -> int:
        return (n + self.page_size - 1) // self.page_size * self.page_size

    def status_after_context(self, ctx) -> BudgetStatus:
        if self.capacity <= 0:
            return BudgetStatus.BUDGET_AVAILABLE
        n = self._aligned(ctx.tokens.active_end)
        if self.used + n > self.capacity:
            return BudgetStatus.BUDGET_EXHAUSTED
        self.used += n
        return BudgetStatus.BUDGET_REACHED if self.used == self.capacity else BudgetStatus.BUDGET_AVAILABLE
