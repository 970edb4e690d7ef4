"""Post-backward gradient finalisation (Megatron-core ``finalize_model_grads``):
data-parallel sync, all-reduce of sequence-parallel-replicated parameter grads (norm weights) over
the tensor-parallel group, shared embedding grads between first and last pipeline stage, router
expert-bias update, per-token loss scaling."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import parallel_state as ps


def _grad_of(p):
    return p.main_grad if hasattr(p, "main_grad") else p.grad


def _allreduce_sequence_parallel_grads(model, config):
    tp = ps.get_tensor_model_parallel_world_size()
    if tp == 1 or not config.sequence_parallel:
        return
    grads = []
    for chunk in model:
        for p in chunk.parameters():
            if p.requires_grad and getattr(p, "sequence_parallel", False):
                g = _grad_of(p)
                if g is not None:
                    grads.append(g)
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=ps.get_tensor_model_parallel_group())
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n


def _allreduce_embedding_grads(model, config):
    if ps.get_pipeline_model_parallel_world_size() == 1 or not ps.is_rank_in_embedding_group(ignore_virtual=True):
        return
    first = model[0]
    last = model[-1]
    chunk = first if ps.is_pipeline_first_stage(ignore_virtual=True) else last
    inner = chunk.module if hasattr(chunk, "module") else chunk
    if not getattr(inner, "share_embeddings_and_output_weights", False):
        return
    w = inner.shared_embedding_or_output_weight()
    g = _grad_of(w)
    if g is not None:
        dist.all_reduce(g, group=ps.get_embedding_group())


def _update_router_expert_bias(model, config):
    if not getattr(config, "moe_router_enable_expert_bias", False):
        return
    for chunk in model:
        for m in chunk.modules():
            if hasattr(m, "update_expert_bias"):
                m.update_expert_bias()


def _return_hot_expert_grads(model, config):
    """--balanced-moe-experts: gradients of the hot experts' replicas go back to the owners (one collective per MoE layer,
    in module order, on every rank)."""
    if not getattr(config, "balanced_moe_experts", False):
        return
    group = ps.get_data_parallel_group(with_context_parallel=True)
    for chunk in model:
        for m in chunk.modules():
            if hasattr(m, "return_hot_grads"):
                buf = getattr(chunk, "_param_to_buffer", {}).get(id(m.experts.weight1)) if hasattr(m.experts, "weight1") else None
                m.return_hot_grads(group, buf.gradient_scaling_factor if buf is not None else 1.0)


def finalize_model_grads(model: List[torch.nn.Module], num_tokens: Optional[torch.Tensor] = None):
    config = (model[0].module if hasattr(model[0], "module") else model[0]).config
    for chunk in model:
        if hasattr(chunk, "finish_grad_sync"):
            chunk.finish_grad_sync()
    _return_hot_expert_grads(model, config)
    _allreduce_sequence_parallel_grads(model, config)
    _allreduce_embedding_grads(model, config)
    _update_router_expert_bias(model, config)
    if num_tokens is not None:
        # per-token loss: gradients were summed over tokens; divide by the global token count
        src = ps.get_pipeline_model_parallel_last_rank()
        if ps.get_pipeline_model_parallel_world_size() > 1:
            dist.broadcast(num_tokens, src=src, group=ps.get_pipeline_model_parallel_group())
        dist.all_reduce(num_tokens, group=ps.get_data_parallel_group(with_context_parallel=True))
        for chunk in model:
            if num_tokens > 0 and hasattr(chunk, "scale_gradients"):
                chunk.scale_gradients(1.0 / num_tokens.item())
