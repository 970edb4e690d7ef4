"""Replica groups: which ranks hold identical copies of the same training state, so that any one healthy member
can write it (reference: mindspeed/core/ttp/replica/replica_group.py:90-491).

With plain data parallelism every DP rank of a (tp, pp) coordinate is a replica.  With the distributed optimizer the
optimizer state is sharded over DP, so replicas only exist between distributed-optimizer *instances*
(``--num-distributed-optimizer-instances`` > 1): rank i of instance a mirrors rank i of instance b."""
from __future__ import annotations

from typing import Dict, List, Sequence, Set

from ..parallel.parallel_state import RankGenerator


def build_replica_groups(world: int, tp: int = 1, pp: int = 1, cp: int = 1, use_distributed_optimizer: bool = False,
                         num_optimizer_instances: int = 1, order: str = "tp-cp-ep-dp-pp") -> List[List[int]]:
    dp = world // (tp * pp * cp)
    gen = RankGenerator(tp=tp, ep=1, dp=dp, pp=pp, cp=cp, order=order)
    groups = []
    for ranks in gen.get_ranks("dp-cp"):
        if not use_distributed_optimizer:
            groups.append(list(ranks))
        else:
            per = len(ranks) // num_optimizer_instances
            for j in range(per):
                groups.append(list(ranks[j::per]))
    return groups


def select_dump_ranks(groups: Sequence[Sequence[int]], faulty: Set[int]) -> Dict[str, object]:
    """Pick the first healthy member of every replica group.  ``ok`` is False when some group lost all its members,
    in which case the state cannot be reconstructed and only a normal restart from the last checkpoint is possible."""
    chosen, lost = [], []
    for g in groups:
        healthy = [r for r in g if r not in faulty]
        if healthy:
            chosen.append(healthy[0])
        else:
            lost.append(list(g))
    return {"ok": not lost, "ranks": sorted(set(chosen)), "lost_groups": lost}
