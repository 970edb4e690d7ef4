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


# ---------------------------------------------------------------------------------------------------------------------
# From command-line arguments to a plan (--automated-pipeline / --automated-pipeline-perf)
# ---------------------------------------------------------------------------------------------------------------------
def analytic_layer_profiles(args, micro_batch_size: Optional[int] = None, peak_flops: float = 1.4e15) -> List[LayerProfile]:
    """Per-layer profile from the model shape alone (no profiling run): GEMM and attention FLOPs at ``peak_flops``, saved
    activations and parameters in bytes, per tensor- / context-parallel rank.  The embedding is charged to the first layer
    and the output layer + loss to the last one, which is what makes an even split uneven in time."""
    mbs = micro_batch_size or args.micro_batch_size
    tp = max(1, getattr(args, "tensor_model_parallel_size", 1))
    cp = max(1, getattr(args, "context_parallel_size", 1))
    s, h = args.seq_length // cp, args.hidden_size
    heads = args.num_attention_heads
    groups = getattr(args, "num_query_groups", None) or heads
    kv = getattr(args, "kv_channels", None) or h // heads
    ffn = getattr(args, "ffn_hidden_size", None) or 4 * h
    gated = 2 if getattr(args, "swiglu", False) else 1
    ne = getattr(args, "num_experts", None)
    topk = getattr(args, "moe_router_topk", 1) or 1
    ep = max(1, getattr(args, "expert_model_parallel_size", 1))
    tokens = mbs * s
    qkv_out = heads * kv + 2 * groups * kv
    attn_params = h * qkv_out + heads * kv * h
    mlp_params = (gated + 1) * h * ffn
    dense_flops = 2 * tokens * (attn_params + mlp_params * (topk if ne else 1)) / tp
    attn_flops = 4 * mbs * s * (args.seq_length) * heads * kv / tp / 2          # causal: half of the square
    fwd = (dense_flops + attn_flops) / peak_flops
    params = (attn_params + (mlp_params * ne / ep if ne else mlp_params)) / tp
    bpe = 2                                                                     # bf16 / fp16 activations
    sp = tp if getattr(args, "sequence_parallel", False) else 1
    act = tokens * bpe * (h * 4 / sp + qkv_out / tp + heads * kv / tp + (gated + 1) * ffn * (topk if ne else 1) / tp)
    layer = LayerProfile(fwd, 2 * fwd, int(act), int(tokens * h * bpe / sp), int(params * bpe))
    out = [dataclasses.replace(layer) for _ in range(args.num_layers)]
    vocab = getattr(args, "padded_vocab_size", None) or getattr(args, "vocab_size", None) or 32000
    head_fwd = 2 * tokens * h * vocab / tp / peak_flops
    out[0] = dataclasses.replace(out[0], param_bytes=out[0].param_bytes + int(vocab * h * bpe / tp))
    last = out[-1]
    out[-1] = dataclasses.replace(last, fwd_time=last.fwd_time + head_fwd, bwd_time=last.bwd_time + 2 * head_fwd,
                                  act_bytes=last.act_bytes + int(tokens * vocab * 4 / tp),
                                  param_bytes=last.param_bytes + int(vocab * h * bpe / tp))
    return out


def plan_from_args(args, budget_bytes: Optional[int] = None, search_micro_batch_size: bool = False) -> Tuple[int, PipelinePlan]:
    """(micro-batch size, plan) for the configured model: layers per pipeline stage and layers to recompute per stage.
    The memory budget is ``--adaptive-recompute-device-size`` (MiB) when given, else 180 GB less the share
    ``--save-memory-ratio`` asks to keep free (10 % when the arguments carry no such value)."""
    pp = args.pipeline_model_parallel_size
    world = getattr(args, "world_size", None) or 1
    dp = max(1, world // (pp * max(1, args.tensor_model_parallel_size) * max(1, getattr(args, "context_parallel_size", 1))))
    if budget_bytes is None:
        mib = getattr(args, "adaptive_recompute_device_size", -1) or -1
        free = float(getattr(args, "save_memory_ratio", 0.1))          # --save-memory-ratio: the share of the device left free
        budget_bytes = int(mib) * (1 << 20) if mib and mib > 0 else int((1.0 - free) * 180e9)
    # bytes of training state per byte of 16-bit parameter: fp32 gradient (2x) + fp32 master and two moments (6x), the
    # latter divided over the data-parallel ranks by the distributed optimizer
    mult = 1.0 + 2.0 + 6.0 / (dp if getattr(args, "use_distributed_optimizer", False) else 1)
    if search_micro_batch_size:
        cands = [m for m in (1, 2, 4, 8) if args.global_batch_size % (m * dp) == 0]
        return search_micro_batch(lambda m: analytic_layer_profiles(args, m), cands, args.global_batch_size, dp, pp, budget_bytes,
                                  state_multiplier=mult)
    n_mb = max(1, args.global_batch_size // (args.micro_batch_size * dp))
    return args.micro_batch_size, solve_pipeline(analytic_layer_profiles(args), pp, n_mb, budget_bytes, state_multiplier=mult)
