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
    def __init__(self, capacity: int, allow_chunking: bool = True, min_chunk: int = 1):
        self.capacity = capacity
        self.used = 0
        self.allow_chunking = allow_chunking
        self.min_chunk = max(1, min_chunk)

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
