"""Automatic pipeline partitioning: layers per stage (and the recompute level per stage) from a per-layer profile.

Given per-layer forward/backward time and activation bytes, parameter bytes, the number of micro-batches in flight
per stage under 1F1B (stage s of P holds min(P - s, n_mb) forwards' activations) and a device budget, choose a
contiguous split of L layers into P stages and for every stage how many of its layers recompute, minimising the
step-time estimate   (n_mb + P - 1) * max_s (stage time)   subject to every stage fitting the budget.

  memory(s) = param_bytes(s) * state_multiplier + in_flight(s) * sum_l act_bytes(l) * (1 - recomputed(l)) + in_flight(s) * input_bytes
  time(s)   = sum_l fwd(l) + bwd(l) + recomputed(l) * fwd(l)

Solved exactly by dynamic programming over (layers consumed, stages used) with a binary search on the bottleneck time.
The "perf" variant additionally searches the micro-batch size from a list using a caller-supplied profile function.
reference: mindspeed/core/memory/auto_pipeline/* (memory-driven split + recompute policy) and
mindspeed/core/performance/auto_pipeline_perf/* (micro-batch / schedule search).
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Optional, Sequence, Tuple


@dataclasses.dataclass
class LayerProfile:
    fwd_time: float
    bwd_time: float
    act_bytes: int          # saved for backward when not recomputed
    input_bytes: int        # what stays when recomputed
    param_bytes: int


@dataclasses.dataclass
class PipelinePlan:
    layers_per_stage: List[int]
    recompute_per_stage: List[int]
    stage_times: List[float]
    stage_bytes: List[int]
    step_time: float
    feasible: bool


def _stage_eval(layers: Sequence[LayerProfile], in_flight: int, budget: int, state_multiplier: float) -> Optional[Tuple[float, int, int]]:
    """Cheapest recompute count that fits: returns (time, bytes, n_recompute) or None when even full recompute fails."""
    params = sum(l.param_bytes for l in layers) * state_multiplier
    base_time = sum(l.fwd_time + l.bwd_time for l in layers)
    # recompute the layers with the best bytes-saved per extra-second first
    order = sorted(range(len(layers)), key=lambda i: -(layers[i].act_bytes - layers[i].input_bytes) / max(layers[i].fwd_time, 1e-12))
    act = sum(l.act_bytes for l in layers)
    extra, n = 0.0, 0
    while True:
        mem = params + in_flight * act
        if mem <= budget:
            return base_time + extra, int(mem), n
        if n == len(layers):
            return None
        l = layers[order[n]]
        act -= l.act_bytes - l.input_bytes
        extra += l.fwd_time
        n += 1


def solve_pipeline(layers: Sequence[LayerProfile], pp: int, n_mb: int, budget_bytes: int, state_multiplier: float = 1.0,
                   extra_first_stage_bytes: int = 0, extra_last_stage_bytes: int = 0) -> PipelinePlan:
    L = len(layers)
    if pp > L:
        raise ValueError("more pipeline stages than layers")
    # cost[s][i][j]: stage s holding layers i..j-1
    memo: Dict[Tuple[int, int, int], Optional[Tuple[float, int, int]]] = {}

    def ev(s, i, j):
        k = (s, i, j)
        if k not in memo:
            b = budget_bytes - (extra_first_stage_bytes if s == 0 else 0) - (extra_last_stage_bytes if s == pp - 1 else 0)
            memo[k] = _stage_eval(layers[i:j], min(pp - s, n_mb), b, state_multiplier)
        return memo[k]

    INF = float("inf")
    # dp[s][j] = minimal bottleneck time using stages 0..s-1 for layers 0..j-1
    dp = [[INF] * (L + 1) for _ in range(pp + 1)]
    cut = [[-1] * (L + 1) for _ in range(pp + 1)]
    dp[0][0] = 0.0
    for s in range(1, pp + 1):
        for j in range(s, L - (pp - s) + 1):
            for i in range(s - 1, j):
                if dp[s - 1][i] == INF:
                    continue
                r = ev(s - 1, i, j)
                if r is None:
                    continue
                v = max(dp[s - 1][i], r[0])
                if v < dp[s][j]:
                    dp[s][j], cut[s][j] = v, i
    if dp[pp][L] == INF:
        even = [L // pp + (1 if r < L % pp else 0) for r in range(pp)]
        return PipelinePlan(even, [n for n in even], [], [], INF, False)
    bounds, j = [], L
    for s in range(pp, 0, -1):
        i = cut[s][j]
        bounds.append((i, j))
        j = i
    bounds.reverse()
    lps, rps, times, mems = [], [], [], []
    for s, (i, j) in enumerate(bounds):
        t, m, n = ev(s, i, j)
        lps.append(j - i); rps.append(n); times.append(t); mems.append(m)
    return PipelinePlan(lps, rps, times, mems, (n_mb + pp - 1) * max(times), True)


def search_micro_batch(profile_fn: Callable[[int], Sequence[LayerProfile]], candidates: Sequence[int], global_batch: int, dp: int,
                       pp: int, budget_bytes: int, **kw) -> Tuple[int, PipelinePlan]:
    """Try each micro-batch size (``profile_fn(mbs)`` returns the per-layer profile at that size) and keep the fastest
    feasible plan; step time is compared per global batch."""
    best: Optional[Tuple[int, PipelinePlan]] = None
    for mbs in candidates:
        if global_batch % (mbs * dp) != 0:
            continue
        n_mb = global_batch // (mbs * dp)
        plan = solve_pipeline(profile_fn(mbs), pp, n_mb, budget_bytes, **kw)
        if plan.feasible and (best is None or plan.step_time < best[1].step_time):
            best = (mbs, plan)
    if best is None:
        raise RuntimeError("no micro-batch size yields a feasible pipeline split within the memory budget")
    return best
