"""Model FLOPs per step and MFU / HFU
(reference: mindspeed/functional/tflops_calculate/adaptor.py:196-231 and Megatron
``num_floating_point_operations``).  MFU counts each forward matmul once (x3 for fwd+bwd); HFU adds
the recomputed forward passes."""
from __future__ import annotations

import json
import os

_PEAKS = None


def measured_peaks():
    """bf16 dense peak per GPU in FLOP/s: the measured cuBLAS figure when the driver left one next to the
    repository, else the nominal Blackwell dense bf16 figure."""
    global _PEAKS
    if _PEAKS is None:
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        path = os.path.join(here, "MEASURED_PEAKS.json")
        _PEAKS = {"bf16_tflops": 2250.0, "bf16_tflops_sustained": 2250.0, "hbm_gbs": 7700.0, "source": "nominal"}
        if os.path.exists(path):
            try:
                with open(path) as f:
                    d = json.load(f)
                _PEAKS.update({k: d[k] for k in ("bf16_tflops", "bf16_tflops_sustained", "hbm_gbs") if k in d})
                _PEAKS["source"] = "measured"
            except Exception:
                pass
    return _PEAKS


def num_floating_point_operations(args, batch_size):
    """Training FLOPs (fwd + bwd) for ``batch_size`` sequences, causal attention counted at half."""
    s, h, L, V = args.seq_length, args.hidden_size, args.num_layers, args.padded_vocab_size or args.vocab_size
    nh = args.num_attention_heads
    ng = args.num_query_groups or nh
    d = args.kv_channels or h // nh
    ffn = args.ffn_hidden_size
    gated = 2 if getattr(args, "swiglu", False) else 1
    tokens = batch_size * s
    if getattr(args, "multi_head_latent_attention", False):
        qd = args.qk_nope_head_dim + args.qk_rope_head_dim
        q_params = (h * args.q_lora_rank + args.q_lora_rank * nh * qd) if args.q_lora_rank else h * nh * qd
        kv_params = h * (args.kv_lora_rank + args.qk_rope_head_dim) + args.kv_lora_rank * nh * (args.qk_nope_head_dim + args.v_head_dim)
        attn_proj = q_params + kv_params + nh * args.v_head_dim * h
        attn_core = 2 * s * nh * (qd + args.v_head_dim) / 2  # per token, causal
    else:
        attn_proj = h * (nh * d + 2 * ng * d) + nh * d * h
        attn_core = 2 * s * nh * d * 2 / 2  # QK^T and PV, per token, causal half
    dense_mlp = h * ffn * gated + ffn * h
    per_layer = []
    ne = getattr(args, "num_experts", None)
    for layer in range(1, L + 1):
        is_moe = ne is not None and layer > getattr(args, "first_k_dense_replace", 0)
        if is_moe:
            mffn = args.moe_ffn_hidden_size or ffn
            mlp = args.moe_router_topk * (h * mffn * gated + mffn * h) + h * ne
            sh = getattr(args, "moe_shared_expert_intermediate_size", None)
            if sh:
                mlp += h * sh * gated + sh * h
        else:
            mlp = dense_mlp
        per_layer.append(2 * (attn_proj + mlp) + attn_core)
    fwd = tokens * (sum(per_layer) + 2 * h * V)
    return 3.0 * fwd


def recompute_extra_flops(args, batch_size):
    if getattr(args, "recompute_granularity", None) != "full":
        return 0.0
    base = num_floating_point_operations(args, batch_size) / 3.0
    s, h, V = args.seq_length, args.hidden_size, args.padded_vocab_size or args.vocab_size
    body = base - batch_size * s * 2 * h * V
    n = args.recompute_num_layers or args.num_layers
    frac = 1.0 if args.recompute_method == "uniform" else min(1.0, n * args.pipeline_model_parallel_size / args.num_layers)
    return body * frac


def mfu(args, batch_size, step_seconds, world_size):
    f = num_floating_point_operations(args, batch_size)
    peak = measured_peaks()["bf16_tflops"] * 1e12
    return f / (step_seconds * world_size * peak)
