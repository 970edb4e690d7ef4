"""Mixture-of-experts layer: router -> dispatch -> grouped experts -> combine (+ shared expert)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import parallel_state as ps
from .experts import GroupedMLP, SequentialMLP, SharedExpertMLP
from .router import TopKRouter
from .token_dispatcher import MoEAllGatherTokenDispatcher, MoEAlltoAllTokenDispatcher


class MoELayer(nn.Module):
    def __init__(self, config, layer_number=1):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        ep = ps.get_expert_model_parallel_world_size()
        if config.num_moe_experts % ep != 0:
            raise ValueError("num_moe_experts must be divisible by the expert parallel size")
        self.num_local_experts = config.num_moe_experts // ep
        off = ps.get_expert_model_parallel_rank() * self.num_local_experts
        self.local_expert_indices = [off + i for i in range(self.num_local_experts)]
        self.router = TopKRouter(config, layer_number)
        if config.moe_grouped_gemm:
            self.experts = GroupedMLP(self.num_local_experts, config)
        else:
            self.experts = SequentialMLP(self.num_local_experts, config)
        kind = config.moe_token_dispatcher_type
        overlap = bool(getattr(config, "moe_alltoall_overlap_comm", False))
        fused = bool(getattr(config, "moe_alltoall_mc2", False)) and config.optimization_level >= 2
        if kind == "allgather":
            self.token_dispatcher = MoEAllGatherTokenDispatcher(self.num_local_experts, self.local_expert_indices, config,
                                                                overlap=bool(getattr(config, "moe_allgather_overlap_comm", False)))
            overlap = overlap or self.token_dispatcher.overlap
        elif kind in ("alltoall", "alltoall_seq"):
            if fused and torch.cuda.is_available():
                from .fused_dispatcher import FusedAlltoAllTokenDispatcher
                self.token_dispatcher = FusedAlltoAllTokenDispatcher(self.num_local_experts, self.local_expert_indices, config)
            else:
                self.token_dispatcher = MoEAlltoAllTokenDispatcher(self.num_local_experts, self.local_expert_indices, config,
                                                                   overlap=overlap)
        else:
            raise ValueError(f"unknown token dispatcher {kind}")
        self.shared_experts = None
        if config.moe_shared_expert_intermediate_size:
            self.shared_experts = SharedExpertMLP(config)
        self.shared_overlap = bool(config.moe_shared_expert_overlap or overlap)
        self._side = None
        # --balanced-moe-experts: the busiest experts are replicated on every expert-parallel rank for one step at a time;
        # their tokens never leave the rank (reference: moe_feature/balanced_moe/modules/moe_layer.py, token_dispatcher.py)
        self.balanced = bool(getattr(config, "balanced_moe_experts", False)) and ep > 1 and bool(config.moe_grouped_gemm)
        self.hot_k = int(getattr(config, "balanced_moe_hot_expert_num", 3) or 0)
        self.hot_groups = int(getattr(config, "trans_hot_expert_group_num", 1) or 1)
        self.hot_experts = []
        self._load = None
        self._hot_w1 = self._hot_w2 = None
        self.unperm_swap = bool(getattr(config, "moe_unperm2_mem_optim_swap", False))
        self.zero_memory = getattr(config, "moe_zero_memory", "disable")
        n_zm = getattr(config, "moe_zero_memory_num_layers", None)
        if n_zm is not None and layer_number > n_zm:
            self.zero_memory = "disable"       # --moe-zero-memory-num-layers: only the first N MoE layers of a stage trade recompute for memory

        # --moe-adaptive-recompute-activation: recompute this layer in backward only on steps where its busiest local expert
        # received more than ``scale`` times the balanced share of tokens (judged by the previous forward; the first one
        # recomputes).  reference: mindspeed/core/transformer/moe/moe_layer.py:59-66, 106-112
        self.adaptive_recompute = bool(getattr(config, "moe_adaptive_recompute_activation", False))
        self.adaptive_scale = float(getattr(config, "moe_adaptive_recompute_activation_scale", 2.0))
        gather = ep * (ps.get_tensor_model_parallel_world_size() if kind == "allgather" and config.sequence_parallel else 1)
        self._share = gather * config.moe_router_topk / config.num_moe_experts        # balanced tokens per expert per local token
        self._max_tokens_per_expert = None
        self.recomputed_steps = 0

    def _recompute_this_step(self, hidden_states) -> bool:
        if not self.adaptive_recompute:
            return False
        if self._max_tokens_per_expert is None:
            return True
        n = hidden_states.shape[0] * hidden_states.shape[1]
        return float(self._max_tokens_per_expert) > n * self._share * self.adaptive_scale

    def _forward(self, hidden_states):
        if hasattr(self.token_dispatcher, "pre_gather"):
            self.token_dispatcher.pre_gather(hidden_states)      # in flight while the router computes
        probs, routing_map = self.router(hidden_states)
        shared = None
        if self.shared_experts is not None and self.shared_overlap and hidden_states.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream()
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                shared = self.shared_experts(hidden_states)
        hot_out = None
        if self.balanced:
            with torch.no_grad():
                cnt = routing_map.sum(0).float()
                self._load = cnt if self._load is None else self._load + cnt
            if self.hot_experts:
                probs, routing_map, hot_out = self._hot_path(hidden_states, probs, routing_map)
        dispatched, tokens_per_expert, pprobs = self.token_dispatcher.token_permutation(hidden_states, probs.to(hidden_states.dtype), routing_map)
        if self.adaptive_recompute:
            with torch.no_grad():
                self._max_tokens_per_expert = torch.as_tensor(tokens_per_expert).max()
        expert_out, _ = self.experts(dispatched, tokens_per_expert, pprobs)
        if self.unperm_swap and self.training and expert_out.is_cuda:
            # --moe-unperm2-mem-optim-swap: what the un-permute saves for backward (the expert output rows) waits in host memory
            from ...memory.host_offload import OffloadSaved
            with OffloadSaved():
                out, _ = self.token_dispatcher.token_unpermutation(expert_out)
        else:
            out, _ = self.token_dispatcher.token_unpermutation(expert_out)
        if hot_out is not None:
            out = out + hot_out
        if self.shared_experts is not None:
            if shared is None:
                shared = self.shared_experts(hidden_states)
            else:
                torch.cuda.current_stream().wait_stream(self._side)
            out = out + shared
        return out

    def _hot_path(self, hidden_states, probs, routing_map):
        """Tokens routed to a hot expert are computed here with the replica of its weights; returns the routing that is left
        for the dispatcher and the hot experts' contribution to the output.  No collective: the replicas were fetched once,
        after the last optimizer step, and their gradients go back to the owners once, after the last micro-batch."""
        from .expert_placement import split_hot_routing
        from .moe_utils import permute, unpermute
        cold_map, cold_probs, hot_map, hot_probs = split_hot_routing(routing_map, probs, self.hot_experts)
        h = hidden_states.reshape(-1, hidden_states.shape[-1])
        rows, order = permute(h, hot_map)
        row_probs = hot_probs.t().contiguous().masked_select(hot_map.t().contiguous()).to(h.dtype)
        y = self.experts.run(rows, hot_map.sum(0).cpu(), row_probs, self._hot_w1, self._hot_w2)
        hot_out = unpermute(y, order, h.shape).view(hidden_states.shape)
        return cold_probs, cold_map, hot_out

    def refresh_hot_experts(self):
        """Once per optimizer step, after the update: choose the ``balanced_moe_hot_expert_num`` busiest experts of the step
        that just ended (token counts summed over the expert-parallel group, so every rank picks the same set) and fetch
        replicas of their new weights."""
        if not self.balanced or self._load is None:
            return self.hot_experts
        import torch.distributed as dist
        from .expert_placement import replicate_hot_experts, select_hot_experts
        group = ps.get_expert_model_parallel_group()
        load = self._load.clone()
        dist.all_reduce(load, group=group)
        self._load = None
        self.hot_experts = select_hot_experts(load, min(self.hot_k, load.numel())) if self.hot_k > 0 else []
        if self.hot_experts:
            with torch.no_grad():
                self._hot_w1 = replicate_hot_experts(self.experts.weight1.data, self.local_expert_indices, self.hot_experts,
                                                     group, self.hot_groups).requires_grad_(True)
                self._hot_w2 = replicate_hot_experts(self.experts.weight2.data, self.local_expert_indices, self.hot_experts,
                                                     group, self.hot_groups).requires_grad_(True)
        return self.hot_experts

    def return_hot_grads(self, group, scale: float):
        """After the data-parallel gradient reduction: sum the replicas' gradients over ``group`` (every rank that holds
        replicas, i.e. the whole data-parallel domain of this layer) and add each hot expert's rows, times ``scale`` (the
        factor the reduction applied to ordinary expert gradients), to its owner's gradient."""
        if not self.hot_experts or self._hot_w1 is None:
            return
        import torch.distributed as dist
        grads = [w.grad if w.grad is not None else torch.zeros_like(w) for w in (self._hot_w1, self._hot_w2)]
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_reduce(flat, group=group)
        n1 = grads[0].numel()
        parts = (flat[:n1].view_as(grads[0]), flat[n1:].view_as(grads[1]))
        for param, g in zip((self.experts.weight1, self.experts.weight2), parts):
            dst = param.main_grad if hasattr(param, "main_grad") else param.grad
            for i, e in enumerate(self.hot_experts):
                if e in self.local_expert_indices and dst is not None:
                    dst[self.local_expert_indices.index(e)].add_((g[i] * scale).to(dst.dtype))
        self._hot_w1.grad = self._hot_w2.grad = None

    def forward(self, hidden_states):
        if self.training and torch.is_grad_enabled() and self._recompute_this_step(hidden_states):
            from ..random import checkpoint
            self.recomputed_steps += 1
            return checkpoint(self._forward, False, hidden_states), None
        if self.training and (self.config.moe_layer_recompute or self.zero_memory != "disable"):
            # zero-memory levels: drop dispatcher intermediates and recompute them in backward
            # (reference: --moe-zero-memory level0/level1, moe_layer_overlap_all2all.py:157-409)
            from ..random import checkpoint
            return checkpoint(self._forward, False, hidden_states), None
        return self._forward(hidden_states), None

    def update_expert_bias(self):
        self.router.update_expert_bias()
