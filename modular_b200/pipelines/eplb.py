"""Expert-parallel load balancing (EPLB): per-expert load statistics, a rebalance plan that
replicates hot experts and packs replicas onto ranks, and the logical-to-physical tables that the
router uses to spread a hot expert's tokens over its replicas.

``EPLBStats`` accumulates token counts per (layer, logical expert) over a sliding window.
``rebalance`` decides, for ``n_physical = n_ranks * slots_per_rank`` physical slots (>= n_logical):
  1. how many replicas each logical expert gets (greedy: repeatedly give one more replica to the
     expert with the largest load per replica),
  2. which rank hosts each replica (longest-processing-time packing: heaviest replica first onto
     the least loaded rank that still has a free slot, never two replicas of an expert on a rank
     while another rank could take it),
and returns ``phy2log [n_physical]``, ``log2phy [n_logical, max_replicas]`` (-1 padded) and
``replica_count [n_logical]``. ``route_to_physical`` maps logical expert ids to physical slot ids,
choosing replicas round-robin by token index.

Reference: max/python/max/pipelines/lib/eplb_stats.py (stats accumulator) and eplb_rebalance.py
(rebalance planner, log2phy tables); the RPC that exposes the stats is serve/pipelines/eplb_stats_rpc.py.
"""

from __future__ import annotations

import heapq
from collections import deque
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch


class EPLBStats:
    def __init__(self, n_layers: int, n_experts: int, window: int = 64):
        self.n_layers, self.n_experts = n_layers, n_experts
        self._window: deque = deque(maxlen=window)
        self._current = np.zeros((n_layers, n_experts), dtype=np.int64)
        self.total_steps = 0

    def record(self, layer: int, topk_ids: torch.Tensor) -> None:
        """Add the routing decisions of one layer of one step (ids of any shape)."""
        ids = topk_ids.reshape(-1)
        counts = torch.bincount(ids[ids >= 0].to(torch.int64), minlength=self.n_experts)[: self.n_experts]
        self._current[layer] += counts.cpu().numpy()

    def end_step(self) -> None:
        self._window.append(self._current)
        self._current = np.zeros_like(self._current)
        self.total_steps += 1

    def load(self) -> np.ndarray:
        """[n_layers, n_experts] tokens routed to each expert over the window."""
        if not self._window:
            return self._current.copy()
        return np.sum(np.stack(list(self._window)), axis=0) + self._current

    def imbalance(self, n_ranks: int) -> np.ndarray:
        """Per layer: max rank load / mean rank load under the contiguous default placement."""
        load = self.load().astype(np.float64)
        per = load.reshape(self.n_layers, n_ranks, -1).sum(-1)
        return per.max(-1) / np.maximum(per.mean(-1), 1e-9)

    def to_dict(self) -> dict:
        return {"steps": self.total_steps, "load": self.load().tolist()}


@dataclass
class RebalancePlan:
    phy2log: np.ndarray        # [n_physical]
    log2phy: np.ndarray        # [n_logical, max_replicas], -1 padded
    replica_count: np.ndarray  # [n_logical]
    rank_load: np.ndarray      # [n_ranks] expected load after rebalancing

    @property
    def imbalance(self) -> float:
        return float(self.rank_load.max() / max(self.rank_load.mean(), 1e-9))


def rebalance(load: np.ndarray, n_ranks: int, slots_per_rank: int) -> RebalancePlan:
    """Plan for one layer. ``load``: [n_logical] tokens per logical expert."""
    load = np.asarray(load, dtype=np.float64)
    n_log, n_phy = load.shape[0], n_ranks * slots_per_rank
    if n_phy < n_log:
        raise ValueError(f"{n_phy} physical slots cannot hold {n_log} experts")
    count = np.ones(n_log, dtype=np.int64)
    heap = [(-load[e], e) for e in range(n_log)]
    heapq.heapify(heap)
    for _ in range(n_phy - n_log):                       # one more replica for the hottest per-replica load
        _, e = heapq.heappop(heap)
        count[e] += 1
        heapq.heappush(heap, (-load[e] / count[e], e))
    replicas = sorted(((load[e] / count[e], e) for e in range(n_log) for _ in range(count[e])), reverse=True)
    rank_load = np.zeros(n_ranks)
    rank_free = np.full(n_ranks, slots_per_rank)
    rank_experts = [set() for _ in range(n_ranks)]
    placement = [[] for _ in range(n_ranks)]
    for w, e in replicas:
        cands = [r for r in range(n_ranks) if rank_free[r] > 0]
        fresh = [r for r in cands if e not in rank_experts[r]]
        r = min(fresh or cands, key=lambda i: (rank_load[i], i))
        placement[r].append(e)
        rank_experts[r].add(e)
        rank_load[r] += w
        rank_free[r] -= 1
    phy2log = np.array([e for r in range(n_ranks) for e in placement[r]], dtype=np.int64)
    log2phy = np.full((n_log, int(count.max())), -1, dtype=np.int64)
    fill = np.zeros(n_log, dtype=np.int64)
    for p, e in enumerate(phy2log):
        log2phy[e, fill[e]] = p
        fill[e] += 1
    return RebalancePlan(phy2log, log2phy, count, rank_load)


def route_to_physical(topk_ids: torch.Tensor, log2phy: torch.Tensor, replica_count: torch.Tensor) -> torch.Tensor:
    """Logical expert ids [T, k] -> physical slot ids, spreading tokens over replicas round-robin."""
    T = topk_ids.shape[0]
    ids = topk_ids.to(torch.int64)
    which = (torch.arange(T, device=ids.device).unsqueeze(1) % replica_count.to(ids.device)[ids])
    return log2phy.to(ids.device)[ids, which].to(topk_ids.dtype)


def gather_expert_weights(w: torch.Tensor, phy2log: np.ndarray, rank: int, slots_per_rank: int) -> torch.Tensor:
    """The physical expert weights rank ``rank`` must hold, from the logical stack ``w [n_logical, ...]``."""
    idx = torch.as_tensor(phy2log[rank * slots_per_rank:(rank + 1) * slots_per_rank], device=w.device)
    return w[idx].contiguous()
