import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def test_planner_balances_and_keeps_experts_in_place():
    from mindspeed_b200.parallel.moe.expert_placement import ExpertPlacementPlanner
    p = ExpertPlacementPlanner(8, 4)
    p.record(torch.tensor([100, 90, 5, 5, 5, 5, 5, 5]))          # rank 0 holds both hot experts
    before = p.imbalance()
    new = p.plan()
    assert sorted(new) == list(range(8))
    assert p.imbalance(new) < 0.5 * before
    moved = sum(1 for a, b in zip(p.placement, new) if a != b)
    assert moved <= 4
    fine = ExpertPlacementPlanner(8, 4, fine_grained_threshold=0.5)
    fine.record(torch.tensor([10, 11, 10, 9, 10, 10, 11, 9]))
    assert fine.plan() == fine.placement                         # already balanced: nothing moves


def _exec(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.parallel.moe.expert_placement import ExpertPlacementExecutor, broadcast_hot_experts
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = dist.new_group(list(range(world)))
    old = [0, 1, 2, 3]
    new = [3, 1, 2, 0]                                            # experts 0 and 3 swap ranks
    per = 2
    w = torch.stack([torch.full((3, 2), float(e)) for e in old[rank * per:(rank + 1) * per]])
    ExpertPlacementExecutor(g).apply([w], old, new)
    got = [int(w[i, 0, 0]) for i in range(per)]
    hot = broadcast_hot_experts(w, new[rank * per:(rank + 1) * per], [0, 2], g)
    dist.destroy_process_group()
    return got, [int(hot[i, 0, 0]) for i in range(2)]


def test_executor_moves_experts_and_hot_broadcast():
    res = run_distributed(_exec, 2)
    assert res[0][0] == [3, 1] and res[1][0] == [2, 0]
    assert res[0][1] == [0, 2] and res[1][1] == [0, 2]


def test_hot_split():
    from mindspeed_b200.parallel.moe.expert_placement import select_hot_experts, split_hot_routing
    rm = torch.tensor([[1, 0, 1, 0], [0, 1, 1, 0], [1, 0, 0, 1]]).bool()
    pr = rm.float() * 0.5
    hot = select_hot_experts(rm.sum(0), 1)
    assert hot == [0] or hot == [2]
    cold_map, cold_p, hot_map, hot_p = split_hot_routing(rm, pr, [2])
    assert cold_map[:, 2].sum() == 0 and hot_map.shape == (3, 1) and hot_map.sum() == 2


def test_fine_grained_threshold_keeps_a_nearly_balanced_placement():
    """With a threshold the planner leaves the placement alone while the heaviest rank is within it of the mean."""
    from mindspeed_b200.parallel.moe.expert_placement import ExpertPlacementPlanner
    load = torch.tensor([100.0, 100.0, 104.0, 100.0, 100.0, 100.0, 100.0, 100.0])
    coarse, fine = ExpertPlacementPlanner(8, 4), ExpertPlacementPlanner(8, 4, fine_grained_threshold=0.08)
    coarse.record(load)
    fine.record(load)
    assert fine.imbalance() < 0.08 and fine.plan() == list(range(8))
    skew = torch.tensor([400.0, 300.0, 10.0, 10.0, 10.0, 10.0, 10.0, 10.0])
    fine.commit(fine.plan())
    fine.record(skew)
    assert fine.imbalance() > 0.08 and fine.plan() != list(range(8))
