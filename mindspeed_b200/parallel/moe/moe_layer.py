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
            self.token_dispatcher = MoEAllGatherTokenDispatcher(self.num_local_experts, self.local_expert_indices, config)
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
        self.zero_memory = getattr(config, "moe_zero_memory", "disable")
        n_zm = getattr(config, "moe_zero_memory_num_layers", None)
        if n_zm is not None and layer_number > n_zm:
            self.zero_memory = "disable"       # --moe-zero-memory-num-layers: only the first N MoE layers of a stage trade recompute for memory

    def _forward(self, hidden_states):
        probs, routing_map = self.router(hidden_states)
        shared = None
        if self.shared_experts is not None and self.shared_overlap and hidden_states.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream()
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                shared = self.shared_experts(hidden_states)
        dispatched, tokens_per_expert, pprobs = self.token_dispatcher.token_permutation(hidden_states, probs.to(hidden_states.dtype), routing_map)
        expert_out, _ = self.experts(dispatched, tokens_per_expert, pprobs)
        out, _ = self.token_dispatcher.token_unpermutation(expert_out)
        if self.shared_experts is not None:
            if shared is None:
                shared = self.shared_experts(hidden_states)
            else:
                torch.cuda.current_stream().wait_stream(self._side)
            out = out + shared
        return out

    def forward(self, hidden_states):
        if self.training and (self.config.moe_layer_recompute or self.zero_memory != "disable"):
            # zero-memory levels: drop dispatcher intermediates and recompute them in backward
            # (reference: --moe-zero-memory level0/level1, moe_layer_overlap_all2all.py:157-409)
            from ..random import checkpoint
            return checkpoint(self._forward, False, hidden_states), None
        return self._forward(hidden_states), None

    def update_expert_bias(self):
        self.router.update_expert_bias()
