"""Expert re-placement and hot-expert replication for load balance across expert-parallel ranks.

* ``ExpertPlacementPlanner``: from accumulated tokens-per-expert, compute a new expert -> rank assignment (each rank
  keeps the same number of experts) that minimises the heaviest rank: longest-processing-time greedy with a capacity
  per rank; a fine-grained mode only moves experts while the max/mean load ratio exceeds a threshold
  (reference: mindspeed/core/transformer/moe/expert_placement/planner.py:58-262, ``--enable-expert-placement``,
  ``--expert-placement-freq``, ``--fine-grained-expert-placement-thre``).
* ``ExpertPlacementExecutor``: applies a plan by exchanging expert weights (and their optimizer state) between ranks
  with one all-to-all per tensor (reference: executor.py:44-586).
* ``select_hot_experts`` / ``split_hot_routing``: replicate the ``k`` hottest experts on every rank so their tokens
  never leave the rank (reference: mindspeed/core/transformer/moe/moe_feature/balanced_moe/*, ``--balanced-moe-experts``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class ExpertPlacementPlanner:
    def __init__(self, num_experts: int, ep_size: int, fine_grained_threshold: Optional[float] = None):
        if num_experts % ep_size:
            raise ValueError("num_experts must divide by the expert parallel size")
        self.E, self.ep, self.per = num_experts, ep_size, num_experts // ep_size
        self.thr = fine_grained_threshold
        self.load = torch.zeros(num_experts, dtype=torch.float64)
        # placement[slot] = expert id held in that slot; slots are rank-major
        self.placement = list(range(num_experts))

    def record(self, tokens_per_expert: torch.Tensor):
        self.load += tokens_per_expert.detach().double().cpu()

    def rank_loads(self, placement=None):
        p = placement or self.placement
        return [float(sum(self.load[e] for e in p[r * self.per:(r + 1) * self.per])) for r in range(self.ep)]

    def imbalance(self, placement=None):
        rl = self.rank_loads(placement)
        mean = sum(rl) / len(rl)
        return (max(rl) / mean - 1.0) if mean > 0 else 0.0

    def plan(self) -> List[int]:
        """New placement (slot -> expert).  Experts that can stay on their rank stay, to minimise traffic."""
        if self.thr is not None and self.imbalance() <= self.thr:
            return list(self.placement)
        order = sorted(range(self.E), key=lambda e: -float(self.load[e]))
        bins: List[List[int]] = [[] for _ in range(self.ep)]
        loads = [0.0] * self.ep
        for e in order:
            r = min((i for i in range(self.ep) if len(bins[i]) < self.per), key=lambda i: loads[i])
            bins[r].append(e)
            loads[r] += float(self.load[e])
        # match new bins to old ranks so that as many experts as possible stay where they are
        old = [set(self.placement[r * self.per:(r + 1) * self.per]) for r in range(self.ep)]
        free = list(range(self.ep))
        assign = {}
        for b in sorted(range(self.ep), key=lambda i: -max(len(set(bins[i]) & o) for o in old)):
            r = max(free, key=lambda rr: len(set(bins[b]) & old[rr]))
            assign[r] = bins[b]
            free.remove(r)
        new = []
        for r in range(self.ep):
            keep = [e for e in self.placement[r * self.per:(r + 1) * self.per] if e in assign[r]]
            rest = [e for e in assign[r] if e not in keep]
            slots = []
            for e in self.placement[r * self.per:(r + 1) * self.per]:
                slots.append(e if e in keep else rest.pop(0))
            new.extend(slots)
        return new

    def commit(self, placement: List[int]):
        self.placement = list(placement)
        self.load.zero_()

    def expert_to_slot(self) -> Dict[int, int]:
        return {e: s for s, e in enumerate(self.placement)}


class ExpertPlacementExecutor:
    """Moves stacked expert tensors [E_local, ...] between expert-parallel ranks according to (old, new) placements."""

    def __init__(self, group):
        self.group = group
        self.ep = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0

    def apply(self, tensors: Sequence[torch.Tensor], old: List[int], new: List[int]):
        per = len(old) // self.ep
        old_slot = {e: s for s, e in enumerate(old)}
        for t in tensors:
            if self.ep == 1:
                src = t.detach().clone()
                with torch.no_grad():
                    for s, e in enumerate(new):
                        t[s].copy_(src[old_slot[e]])
                continue
            # rows I send to each rank (in the receiver's slot order) and rows I receive
            send, send_counts = [], []
            for dst in range(self.ep):
                rows = [old_slot[e] - self.rank * per for e in new[dst * per:(dst + 1) * per] if old_slot[e] // per == self.rank]
                send.append(t.detach()[rows] if rows else t.detach()[:0])
                send_counts.append(len(rows))
            recv_counts = [sum(1 for e in new[self.rank * per:(self.rank + 1) * per] if old_slot[e] // per == src) for src in range(self.ep)]
            from .. import mappings as M
            flat = torch.cat(send, dim=0).reshape(sum(send_counts), -1)
            got = M.all_to_all_single(flat, self.group, recv_counts, send_counts)
            # received rows are grouped by source rank, each group in my slot order restricted to that source
            pos = {src: 0 for src in range(self.ep)}
            starts, acc = {}, 0
            for src in range(self.ep):
                starts[src] = acc
                acc += recv_counts[src]
            with torch.no_grad():
                out = torch.empty_like(t)
                for s, e in enumerate(new[self.rank * per:(self.rank + 1) * per]):
                    src = old_slot[e] // per
                    out[s].copy_(got[starts[src] + pos[src]].view(t.shape[1:]))
                    pos[src] += 1
                t.copy_(out)


def select_hot_experts(tokens_per_expert: torch.Tensor, k: int) -> List[int]:
    return torch.topk(tokens_per_expert.float(), k).indices.sort().values.tolist()


def split_hot_routing(routing_map: torch.Tensor, probs: torch.Tensor, hot: Sequence[int]):
    """(cold_map, cold_probs, hot_map, hot_probs): tokens routed to hot experts are handled by the local replicas."""
    hot_mask = torch.zeros(routing_map.shape[1], dtype=torch.bool, device=routing_map.device)
    hot_mask[list(hot)] = True
    cold_map = routing_map & ~hot_mask
    hot_map = routing_map[:, hot_mask]
    return cold_map, probs * cold_map, hot_map, probs[:, hot_mask] * hot_map


def broadcast_hot_experts(stacked: torch.Tensor, local_ids: Sequence[int], hot: Sequence[int], group) -> torch.Tensor:
    """Gather the weights of the hot experts from their owners: returns [len(hot), ...] on every rank."""
    out = torch.zeros(len(hot), *stacked.shape[1:], dtype=stacked.dtype, device=stacked.device)
    for i, e in enumerate(hot):
        if e in local_ids:
            out[i].copy_(stacked[list(local_ids).index(e)])
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(out, group=group)     # exactly one rank contributes each row
    return out


def replicate_hot_experts(stacked: torch.Tensor, local_ids: Sequence[int], hot: Sequence[int], group, n_groups: int = 1) -> torch.Tensor:
    """[len(hot), ...] copies of the hot experts' rows of ``stacked`` on every rank of ``group`` (each row is contributed by
    its one owner).  ``n_groups`` collectives instead of one, so the first replicas are usable while the rest is in flight."""
    out = torch.zeros(len(hot), *stacked.shape[1:], dtype=stacked.dtype, device=stacked.device)
    local_ids = list(local_ids)
    for i, e in enumerate(hot):
        if e in local_ids:
            out[i].copy_(stacked[local_ids.index(e)])
    if group is not None and dist.get_world_size(group) > 1:
        works = [dist.all_reduce(c, group=group, async_op=True) for c in out.chunk(max(1, min(n_groups, len(hot))), 0)]
        for w in works:
            w.wait()
    return out
