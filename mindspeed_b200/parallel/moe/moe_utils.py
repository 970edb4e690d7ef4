"""MoE helpers: permutation, chunk sorting, load-balancing losses, aux-loss gradient scaler.

``permute`` / ``unpermute`` follow Megatron-core's routing-map form: tokens are gathered expert-major according to a
boolean map [tokens, experts]; ``unpermute`` scatters back weighted by the router probabilities.  On a GPU at
optimisation level >= 1 the gather / weighted scatter-add run as the hand-written kernels in
mindspeed_b200/ops/permute.py (reference: mindspeed/core/fusions/fused_moe_permute.py:50-84,
mindspeed/ops/csrc/cann/npu_moe_token_permute.cpp).
"""
from __future__ import annotations

from typing import List, Optional

import torch


def permute(tokens, routing_map, num_out_tokens: Optional[int] = None, fused: bool = False):
    """tokens [T, H]; routing_map [T, E] bool -> (permuted [T*topk, H] expert-major, sorted_indices [T*topk])."""
    T, _ = tokens.shape
    E = routing_map.shape[1]
    rm = routing_map.bool().t().contiguous()  # [E, T]
    token_indices = torch.arange(T, device=tokens.device).unsqueeze(0).expand(E, -1)
    sorted_indices = token_indices.masked_select(rm)
    if num_out_tokens is not None:
        sorted_indices = sorted_indices[:num_out_tokens]
    if fused and tokens.is_cuda:
        from ...ops.permute import gather_rows
        return gather_rows(tokens, sorted_indices), sorted_indices
    return tokens.index_select(0, sorted_indices), sorted_indices


def unpermute(permuted_tokens, sorted_indices, restore_shape, probs=None, routing_map=None, fused: bool = False):
    """Inverse of ``permute``; with ``probs`` [T, E] each copy is weighted by its router probability."""
    T, H = restore_shape
    w = None
    if probs is not None:
        w = probs.t().contiguous().masked_select(routing_map.bool().t().contiguous())
    if fused and permuted_tokens.is_cuda:
        from ...ops.permute import scatter_add_rows
        return scatter_add_rows(permuted_tokens, sorted_indices, T, w)
    if w is not None:
        permuted_tokens = permuted_tokens * w.unsqueeze(-1).to(permuted_tokens.dtype)
    out = torch.zeros(T, H, dtype=permuted_tokens.dtype, device=permuted_tokens.device)
    out.scatter_add_(0, sorted_indices.unsqueeze(1).expand(-1, H), permuted_tokens)
    return out


def sort_chunks_by_idxs(x, split_sizes, sorted_idxs, probs=None):
    """Split ``x`` along dim 0 into chunks of ``split_sizes`` and concatenate them in ``sorted_idxs`` order
    (reference Triton version: mindspeed/ops/triton/sort_chunks_by_idx.py:24,119)."""
    sizes = split_sizes.tolist() if torch.is_tensor(split_sizes) else list(split_sizes)
    order = sorted_idxs.tolist() if torch.is_tensor(sorted_idxs) else list(sorted_idxs)
    chunks = torch.split(x, sizes, dim=0)
    out = torch.cat([chunks[i] for i in order], dim=0)
    if probs is not None:
        pc = torch.split(probs, sizes, dim=0)
        return out, torch.cat([pc[i] for i in order], dim=0)
    return out


def switch_load_balancing_loss_func(probs, tokens_per_expert, topk, moe_aux_loss_coeff, num_tokens=None):
    """E * sum_e f_e * P_e scaled by coeff / topk (Switch-transformer form used by Megatron-core)."""
    T = probs.shape[0] if num_tokens is None else num_tokens
    E = probs.shape[1]
    aggregated = probs.sum(dim=0)
    return torch.sum(aggregated * tokens_per_expert) * (E * moe_aux_loss_coeff / (T * T * topk))


def sequence_load_balancing_loss_func(probs, routing_map, batch_size, seq_length, topk, moe_aux_loss_coeff):
    E = probs.shape[1]
    p = probs.view(seq_length, batch_size, E).sum(0)  # [b, E]
    f = routing_map.view(seq_length, batch_size, E).sum(0).float()
    return torch.sum(p * f) * (E * moe_aux_loss_coeff / (seq_length * seq_length * topk * batch_size))


def z_loss_func(logits, z_loss_coeff):
    return torch.mean(torch.square(torch.logsumexp(logits, dim=-1))) * z_loss_coeff


class MoEAuxLossAutoScaler(torch.autograd.Function):
    """Identity on the activations that adds d(aux_loss) to the graph with an adjustable scale."""
    main_loss_backward_scale = None

    @staticmethod
    def forward(ctx, output, aux_loss):
        ctx.save_for_backward(aux_loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (aux_loss,) = ctx.saved_tensors
        scale = MoEAuxLossAutoScaler.main_loss_backward_scale
        if scale is None:
            scale = torch.tensor(1.0, device=aux_loss.device)
        return grad_output, torch.ones_like(aux_loss) * scale.to(aux_loss.device)

    @staticmethod
    def set_loss_scale(scale):
        MoEAuxLossAutoScaler.main_loss_backward_scale = scale if torch.is_tensor(scale) else torch.tensor(float(scale))


def topk_softmax_with_capacity(logits, topk, capacity_factor=None, pad_to_capacity=False, drop_policy="probs",
                               use_pre_softmax=False, num_groups=None, group_topk=None, scaling_factor=None,
                               score_function="softmax", expert_bias=None, deterministic_mode=False):
    """Returns (probs [T, E] with zeros for unrouted experts, routing_map [T, E] bool, tokens_per_expert [E])."""
    T, E = logits.shape

    def pick(scores):
        if group_topk:
            g = scores.view(T, num_groups, E // num_groups)
            gscore = g.topk(max(1, topk // group_topk), dim=-1)[0].sum(-1)
            gidx = gscore.topk(group_topk, dim=-1)[1]
            gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1).unsqueeze(-1).expand_as(g).reshape(T, E)
            scores = scores.masked_fill(~gmask.bool(), float("-inf"))
        return scores.topk(topk, dim=1)

    if score_function == "softmax":
        if use_pre_softmax:
            scores = torch.softmax(logits.float(), dim=-1).type_as(logits)
            vals, idx = pick(scores)
        else:
            vals, idx = pick(logits)
            vals = torch.softmax(vals.float(), dim=-1).type_as(logits)
    elif score_function == "sigmoid":
        scores = torch.sigmoid(logits.float())
        if expert_bias is not None:
            _, idx = pick(scores + expert_bias)
            vals = scores.gather(1, idx)
        else:
            vals, idx = pick(scores)
        if topk > 1:
            vals = vals / (vals.sum(dim=-1, keepdim=True) + 1e-20)
        vals = vals.type_as(logits)
    else:
        raise ValueError(f"unknown score function {score_function}")
    if scaling_factor:
        vals = vals * scaling_factor
    probs = torch.zeros_like(logits).scatter(1, idx, vals)
    routing_map = torch.zeros_like(logits, dtype=torch.int32).scatter(1, idx, 1).bool()
    if capacity_factor is not None:
        cap = int(max(1, (T * topk * capacity_factor + E - 1) // E))
        if drop_policy == "probs":
            _, keep = torch.topk(probs, k=min(cap, T), dim=0, sorted=False)
            cmask = torch.zeros_like(logits, dtype=torch.bool).scatter(0, keep, True)
        else:
            _, keep = torch.topk(routing_map.int(), k=min(cap, T), dim=0, sorted=False)
            cmask = torch.zeros_like(logits, dtype=torch.bool).scatter(0, keep, True)
        if pad_to_capacity:
            routing_map, probs = cmask, probs * cmask
        else:
            routing_map = routing_map & cmask
            probs = probs * routing_map
    tokens_per_expert = routing_map.sum(dim=0)
    return probs, routing_map, tokens_per_expert


def reduce_moe_metrics(tracker, calls_per_layer: int, clear: bool = True):
    """{name: per-layer means [num_layers]} of what ``track_moe_metrics`` accumulated since the last call: layers live on
    different pipeline stages (summed over the pipeline group), every layer added one value per forward (``calls_per_layer``
    = micro-batches x steps) and data-parallel ranks see different tokens (averaged).  Collective over the pipeline and
    data-parallel groups: every rank must call it (reference: Megatron ``reduce_aux_losses_tracker_across_ranks`` as used by
    mindspeed/core/transformer/moe/moe_utils.py track_moe_metrics)."""
    import torch.distributed as dist
    from .. import parallel_state as ps
    out = {}
    for name in sorted(tracker):
        v = tracker[name]["values"].float().clone() / max(1, calls_per_layer)
        if dist.is_initialized() and ps.model_parallel_is_initialized():
            if ps.get_pipeline_model_parallel_world_size() > 1:
                dist.all_reduce(v, group=ps.get_pipeline_model_parallel_group())
            if ps.get_data_parallel_world_size() > 1:
                dist.all_reduce(v, group=ps.get_data_parallel_group())
                v /= ps.get_data_parallel_world_size()
        out[name] = v
        if clear:
            tracker[name]["values"].zero_()
    return out


def track_moe_metrics(tracker, name, value, layer_number, num_layers):
    if name not in tracker:
        tracker[name] = {"values": torch.zeros(num_layers, device=value.device)}
    tracker[name]["values"][layer_number - 1] += value.detach()
