"""White-box memory and time models.

Memory = static (parameters, gradients, optimizer state by dtype and sharding) + activations (per layer, by
sequence / tensor / context sharding and recompute).  Time follows the reference's composition
(mindspeed/auto_settings/module/time_cost.py:36-80):
    micro_batches = gbs / (dp * mbs);  bubble = (pp - 1) / (micro_batches * vpp + pp - 1)
    total = (layer_time * layers_per_stage * micro_batches + exposed_comm) / (1 - bubble) + dp_time + optimizer_time
with two changes for this machine: communication per parallel dimension is ``latency + bytes / measured bandwidth``
instead of a fitted line over profiled samples, and a fused GEMM+collective costs max(compute, comm) instead of the sum.
"""
from __future__ import annotations

from dataclasses import dataclass

from .hardware import Hardware
from .search_space import ModelDesc, SearchConfig

GEMM_EFF = 0.80          # fraction of the cuBLAS peak the tensor-parallel shard shapes reach
ATTN_EFF = 0.55


@dataclass
class Estimate:
    config: SearchConfig
    memory_gib: float
    step_ms: float
    fits: bool
    detail: dict


def memory_gib(m: ModelDesc, c: SearchConfig) -> dict:
    attn, mlp = m.dense_params_per_layer()
    exp = m.expert_params_per_layer()
    layers = m.num_layers // c.pp
    dense_layer = (attn + (0 if exp else mlp)) / c.tp
    expert_layer = exp / c.ep if exp else 0
    emb = m.vocab_size * m.hidden_size / c.tp
    n_emb = (1 if c.pp > 1 else 2)      # first / last stage hold one each
    dense = dense_layer * layers + emb * n_emb
    expert = expert_layer * layers
    shard = c.dp * c.cp if c.use_distributed_optimizer else 1
    eshard = max(1, c.dp * c.cp // c.ep) if c.use_distributed_optimizer else 1
    static = dense * (2 + 4) + expert * (2 + 4) + dense * 12 / shard + expert * 12 / eshard
    s = m.seq_length / c.cp
    sp = c.tp if c.sequence_parallel else 1
    h, f = m.hidden_size, (m.moe_ffn_hidden_size or m.ffn_hidden_size) if exp else m.ffn_hidden_size
    topk = m.moe_topk if exp else 1
    # saved per layer (bytes per token): sharded residual/norm tensors + tensor-parallel ones
    per_tok = (4 * h / sp + (m.num_attention_heads + 2 * m.num_query_groups) * m.kv_channels / c.tp + h / c.tp * 1
               + topk * (3 if m.gated else 2) * f / c.tp) * 2
    act_layer = per_tok * s * c.mbs
    kept = layers - c.recompute_layers
    in_flight = min(c.pp, m.global_batch_size // (c.dp * c.mbs)) if c.pp > 1 else 1
    act = (act_layer * kept + 2 * h * s * c.mbs / sp * c.recompute_layers) * in_flight + act_layer  # + one layer being recomputed
    logits = s * c.mbs * m.vocab_size / c.tp * (2 + 4)
    gib = 1024 ** 3
    return {"static": static / gib, "activations": act / gib, "logits": logits / gib, "total": (static + act + logits) / gib + 4.0}


def layer_work(m: ModelDesc, c: SearchConfig) -> dict:
    """FLOPs and communicated bytes of ONE layer's forward for one micro-batch on one rank."""
    attn, mlp = m.dense_params_per_layer()
    exp = m.expert_params_per_layer()
    s = m.seq_length
    tokens = s * c.mbs / c.cp
    mlp_flops = (exp / m.num_experts * m.moe_topk if exp else mlp)
    return {"tokens": tokens,
            "gemm_flops": 2 * tokens * (attn + mlp_flops) / c.tp,
            "attn_flops": 2 * 2 * tokens * s * m.num_attention_heads * m.kv_channels / 2 / c.tp,
            # 2 all-gathers + 2 reduce-scatters of the hidden activation; bytes that cross the links per GPU, each
            "tp_bytes": tokens * m.hidden_size * 2 * (c.tp - 1) / c.tp if c.tp > 1 else 0.0,
            "cp_bytes": 2 * tokens * m.num_query_groups * m.kv_channels * 2 / c.tp if c.cp > 1 else 0.0,
            "ep_bytes": tokens * m.moe_topk * m.hidden_size * 2 * (c.ep - 1) / c.ep if (exp and c.ep > 1) else 0.0}


def step_ms(m: ModelDesc, c: SearchConfig, hw: Hardware, db=None, comm=None) -> dict:
    """``db`` (operator_db.OperatorDB) replaces the fixed GEMM / attention efficiencies by what was measured; ``comm``
    (comm_predictors.CommPredictors) replaces latency + bytes / bandwidth by the fitted per-dimension lines."""
    attn, mlp = m.dense_params_per_layer()
    exp = m.expert_params_per_layer()
    s = m.seq_length
    w = layer_work(m, c)
    tokens, gemm_f, attn_f = w["tokens"], w["gemm_flops"], w["attn_flops"]
    peak = hw.bf16_tflops * 1e12
    gemm_eff = (db.efficiency("gemm", peak) if db is not None else None) or GEMM_EFF
    attn_eff = (db.efficiency("attention", peak) if db is not None else None) or ATTN_EFF
    fwd = gemm_f / (peak * gemm_eff) + attn_f / (peak * attn_eff)
    tp_bytes = w["tp_bytes"]
    link = hw.nvlink_gbs * 1e9
    fused = c.tp > 1 and c.fused_tp_comm and c.sequence_parallel
    if comm is not None and c.tp > 1:
        dim = "mc2" if fused else "tp"
        tp_comm = 4 * comm.time(dim, tp_bytes, c.tp)
        layer_fwd = fwd + 4 * comm.time(dim, tp_bytes, c.tp, exposed=True)
        if fused:
            layer_fwd = max(layer_fwd, tp_comm)
    else:
        tp_comm = 4 * (tp_bytes / link + hw.collective_latency_us * 1e-6) if c.tp > 1 else 0.0
        if fused:
            layer_fwd = max(fwd, tp_comm) + 0.15 * min(fwd, tp_comm)    # fused: overlapped up to pipeline fill / drain
        else:
            layer_fwd = fwd + tp_comm
    cp_comm = 0.0
    if c.cp > 1:
        kv_bytes = w["cp_bytes"]
        if comm is not None:
            cp_comm = (c.cp - 1) * comm.time("cp", kv_bytes, c.cp, exposed=True)
        else:
            cp_comm = max(0.0, (c.cp - 1) * kv_bytes / link - attn_f / (peak * attn_eff))   # ring steps hide behind attention
    ep_comm = 0.0
    if exp and c.ep > 1:
        if comm is not None:
            ep_comm = 2 * comm.time("ep", w["ep_bytes"], c.ep, exposed=True)
        else:
            ep_comm = 2 * w["ep_bytes"] / link + 2 * hw.collective_latency_us * 1e-6
    layer = 3 * layer_fwd + 3 * (cp_comm + ep_comm)
    layers = m.num_layers // c.pp
    recompute = layer_fwd * c.recompute_layers
    n_mb = m.global_batch_size // (c.dp * c.mbs)
    head = 3 * 2 * tokens * m.hidden_size * m.vocab_size / c.tp / (peak * GEMM_EFF) / c.pp
    per_mb = layer * layers + recompute + head
    bubble = (c.pp - 1) / (n_mb * c.vpp + c.pp - 1) if c.pp > 1 else 0.0
    pp_comm = 2 * n_mb * (tokens * m.hidden_size * 2 / (c.tp if c.sequence_parallel else 1) / link + hw.p2p_latency_us * 1e-6) if c.pp > 1 else 0.0
    params_local = (attn + (0 if exp else mlp)) / c.tp * layers + exp / max(c.ep, 1) * layers
    dp_comm = 0.0
    if c.dp * c.cp > 1:
        bw = (hw.allreduce_bus_gbs if c.tp * c.cp * c.pp * c.dp <= hw.gpus_per_node else hw.internode_gbs) * 1e9
        dp_comm = 0.3 * (params_local * 4 * 2 / bw)         # reduce-scatter + all-gather, mostly overlapped with backward
    shard = c.dp * c.cp if c.use_distributed_optimizer else 1
    opt = params_local / shard * 30 / (hw.hbm_gbs * 1e9)
    total = (per_mb * n_mb + pp_comm) / (1 - bubble) + dp_comm + opt
    return {"per_microbatch_ms": per_mb * 1e3, "bubble": bubble, "tp_comm_ms": tp_comm * 1e3, "total_ms": total * 1e3}


def estimate(m: ModelDesc, c: SearchConfig, hw: Hardware, db=None, comm=None) -> Estimate:
    mem = memory_gib(m, c)
    t = step_ms(m, c, hw, db, comm)
    return Estimate(c, mem["total"], t["total_ms"], mem["total"] <= hw.hbm_gib, {**mem, **t})


def learn_from_profile(summary, m: ModelDesc, c: SearchConfig, hw: Hardware, db, comm, steps: int = 1):
    """Feed one profiled run of configuration ``c`` (``profiling_parse.ProfileSummary`` over ``steps`` optimizer steps) into
    the operator database and the communication predictors: achieved GEMM / attention throughput for the shapes of this
    configuration, and one (traffic, total time, exposed time) sample per communication class that appears."""
    w = layer_work(m, c)
    layers = m.num_layers // c.pp
    n_mb = m.global_batch_size // (c.dp * c.mbs)
    calls = 3 * layers * n_mb * steps                       # forward + two backward GEMM passes per layer and micro-batch
    ops = summary.ops
    if "gemm" in ops or "tp_fused" in ops:
        us = ops.get("gemm", None).total_us if "gemm" in ops else 0.0
        us += ops["tp_fused"].total_us if "tp_fused" in ops else 0.0      # the fused kernels do the layer GEMMs
        db.record("gemm", (int(w["tokens"]), m.hidden_size, c.tp), us / 1e3 / calls, flops=w["gemm_flops"])
    if "attention" in ops:
        db.record("attention", (int(w["tokens"]), m.seq_length, m.num_attention_heads // c.tp), ops["attention"].total_us / 1e3 / calls,
                  flops=w["attn_flops"])
    per_call = {"tp_fused": ("mc2", w["tp_bytes"], c.tp, 4 * calls), "ep_a2a": ("ep", w["ep_bytes"], c.ep, 2 * calls),
                "p2p": ("pp" if c.pp > 1 else "cp", w["tokens"] * m.hidden_size * 2 if c.pp > 1 else w["cp_bytes"],
                        c.pp if c.pp > 1 else c.cp, max(1, 2 * n_mb * steps if c.pp > 1 else (c.cp - 1) * calls))}
    for cls, (dim, nbytes, span, n) in per_call.items():
        if cls in ops and nbytes > 0 and span > 1:
            comm.add_sample(dim, nbytes, span, ops[cls].total_us * 1e-6 / n, ops[cls].exposed_us * 1e-6 / n)
    comm.fit()
