"""Expert parallelism for HF-style sparse blocks: ``dispatch -> local experts -> combine``.

A block is expected to expose ``gate`` (or ``router``): Linear(hidden -> num_experts), ``experts``: ModuleList of
per-expert MLPs, and ``top_k`` (or ``num_experts_per_tok``).  ``shard_experts`` keeps only the local experts on each
expert-parallel rank and swaps the block's forward for an all-to-all dispatch around them; routing follows the
common HF recipe (softmax over all experts, top-k, renormalise).
reference: mindspeed/fsdp/distributed/expert_parallel/dispatcher.py:11-113 (dispatch_mlp_combine).
"""
from __future__ import annotations

import types
from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel import mappings as M
from ..parallel.moe.moe_utils import permute, sort_chunks_by_idxs, unpermute
from ..utils.patterns import match as _match


def dispatch_mlp_combine(x: torch.Tensor, probs: torch.Tensor, routing_map: torch.Tensor, local_experts: nn.ModuleList,
                         ep_group) -> torch.Tensor:
    """x [T, H]; probs / routing_map [T, E].  Returns sum_k p_k * expert_k(x) with experts spread over ``ep_group``."""
    ep, me = M._ws(ep_group), M._rk(ep_group)
    T, H = x.shape
    E = routing_map.shape[1]
    E_loc = E // ep
    permuted, sorted_idx = permute(x, routing_map)
    counts = routing_map.sum(0).to(torch.int64)
    if ep > 1:
        allc = [torch.empty_like(counts) for _ in range(ep)]
        dist.all_gather(allc, counts, group=ep_group)
        allc = torch.stack(allc).cpu()                                 # [ep, E]
        in_splits = allc[me].view(ep, E_loc).sum(1).tolist()
        per_src = allc[:, me * E_loc:(me + 1) * E_loc]                  # [ep, E_loc]
        out_splits = per_src.sum(1).tolist()
        recv = M.all_to_all(ep_group, permuted, out_splits, in_splits)
        chunk_sizes = per_src.reshape(-1).tolist()
        fwd = torch.arange(ep * E_loc).view(ep, E_loc).t().reshape(-1).tolist()
        bwd = torch.arange(ep * E_loc).view(E_loc, ep).t().reshape(-1).tolist()
        if E_loc > 1:
            recv = sort_chunks_by_idxs(recv, chunk_sizes, fwd)
        tokens_per_expert = per_src.sum(0).tolist()
    else:
        recv, tokens_per_expert = permuted, counts.cpu().tolist()
    outs, start = [], 0
    for e, n in enumerate(tokens_per_expert):
        seg = recv[start:start + n]
        outs.append(local_experts[e](seg))      # also for n == 0: keeps hooks and (zero) gradients of idle experts regular
        start += n
    y = torch.cat(outs, dim=0) if outs else recv
    if ep > 1:
        if E_loc > 1:
            y = sort_chunks_by_idxs(y, [chunk_sizes[i] for i in fwd], bwd)
        y = M.all_to_all(ep_group, y, in_splits, out_splits)
    return unpermute(y, sorted_idx, (T, H), probs=probs, routing_map=routing_map)


def _ep_forward(self, hidden_states):
    shape = hidden_states.shape
    x = hidden_states.reshape(-1, shape[-1])
    gate = getattr(self, "gate", None) or getattr(self, "router")
    logits = gate(x).float()
    scores = torch.softmax(logits, dim=-1)
    topv, topi = scores.topk(self._ep_top_k, dim=-1)
    topv = topv / topv.sum(-1, keepdim=True)
    probs = torch.zeros_like(scores).scatter(1, topi, topv).to(x.dtype)
    routing_map = torch.zeros_like(scores, dtype=torch.bool).scatter(1, topi, True)
    out = dispatch_mlp_combine(x, probs, routing_map, self.experts, self._ep_group)
    return out.view(shape)


def shard_experts(model: nn.Module, patterns: List[str], ep_group) -> int:
    """Keep the local experts of every matching block and install the dispatching forward; returns blocks changed."""
    ep, me = M._ws(ep_group), M._rk(ep_group)
    changed = 0
    for name, mod in list(model.named_modules()):
        if not any(_match(name, p) or type(mod).__name__ == p for p in patterns):
            continue
        experts = getattr(mod, "experts", None)
        if not isinstance(experts, nn.ModuleList):
            raise TypeError(f"{name}: expected an 'experts' ModuleList")
        E = len(experts)
        if E % ep != 0:
            raise ValueError(f"{name}: {E} experts not divisible by expert parallel size {ep}")
        E_loc = E // ep
        mod.experts = nn.ModuleList([experts[i] for i in range(me * E_loc, (me + 1) * E_loc)])
        for p in mod.experts.parameters():
            p.allreduce = False            # expert parameters are reduced over the expert-data-parallel group only
        mod._ep_group = ep_group
        mod._ep_top_k = int(getattr(mod, "top_k", None) or getattr(mod, "num_experts_per_tok", 2))
        mod.forward = types.MethodType(_ep_forward, mod)
        changed += 1
    return changed
