"""EPLB: statistics, replica planning, and routing through the physical tables."""

import numpy as np
import torch

from modular_b200.pipelines.eplb import EPLBStats, gather_expert_weights, rebalance, route_to_physical


def test_stats_window_and_imbalance():
    st = EPLBStats(n_layers=2, n_experts=8, window=2)
    for step in range(3):
        st.record(0, torch.tensor([[0, 1], [0, 2], [0, 3]]))
        st.record(1, torch.tensor([4, 5, 6, 7, -1]))
        st.end_step()
    load = st.load()
    assert load[0, 0] == 6 and load[0, 1] == 2 and load[1, 4:].tolist() == [2, 2, 2, 2]     # window of 2 steps
    imb = st.imbalance(n_ranks=2)
    assert imb[0] == 2.0 and imb[1] == 2.0       # layer 0: all load on rank 0; layer 1: all on rank 1
    assert st.to_dict()["steps"] == 3


def test_rebalance_replicates_hot_experts_and_balances_ranks():
    load = np.array([1000, 10, 10, 10, 10, 10, 10, 10], dtype=np.float64)
    plan = rebalance(load, n_ranks=4, slots_per_rank=3)           # 12 slots for 8 experts
    assert plan.replica_count[0] == 5 and plan.replica_count.sum() == 12
    assert sorted(plan.phy2log.tolist()).count(0) == 5
    for r in range(4):      # replicas of the hot expert sit on different ranks where possible
        assert plan.phy2log[r * 3:(r + 1) * 3].tolist().count(0) <= 2
    before = load.reshape(4, 2).sum(1)
    assert plan.imbalance < 1.6 < before.max() / before.mean()      # 5 replicas of 200 over 4 ranks: one rank holds two
    for e in range(8):
        phys = [p for p in plan.log2phy[e] if p >= 0]
        assert len(phys) == plan.replica_count[e] and all(plan.phy2log[p] == e for p in phys)


def test_routing_spreads_tokens_and_weights_follow_plan():
    load = np.array([100, 1, 1, 1], dtype=np.float64)
    plan = rebalance(load, n_ranks=2, slots_per_rank=3)
    ids = torch.tensor([[0, 1]] * 6 + [[2, 3]])
    phys = route_to_physical(ids, torch.from_numpy(plan.log2phy), torch.from_numpy(plan.replica_count))
    assert torch.equal(torch.from_numpy(plan.phy2log)[phys], ids.long())                 # same logical experts
    assert len(set(phys[:6, 0].tolist())) == plan.replica_count[0]                         # all replicas used
    w = torch.arange(4).float().view(4, 1, 1).expand(4, 2, 2)
    local = gather_expert_weights(w, plan.phy2log, rank=1, slots_per_rank=3)
    assert local[:, 0, 0].long().tolist() == plan.phy2log[3:6].tolist()
