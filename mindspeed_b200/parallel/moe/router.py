"""Top-k router with softmax / sigmoid scores, group-limited routing, expert bias and load-balancing losses
(Megatron-core ``TopKRouter`` surface; reference adjustments mindspeed/core/transformer/moe/router.py:71-107)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import parallel_state as ps
from .moe_utils import (MoEAuxLossAutoScaler, sequence_load_balancing_loss_func, switch_load_balancing_loss_func,
                        topk_softmax_with_capacity, track_moe_metrics, z_loss_func)


class TopKRouter(nn.Module):
    def __init__(self, config, layer_number=1):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        self.num_experts, self.topk = config.num_moe_experts, config.moe_router_topk
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.empty(self.num_experts, config.hidden_size, device=dev, dtype=torch.float32))
        if config.perform_initialization:
            with torch.no_grad():
                w = torch.empty(self.num_experts, config.hidden_size)
                config.init_method(w)
                self.weight.copy_(w)
        setattr(self.weight, "sequence_parallel", config.sequence_parallel)
        self.score_function = config.moe_router_score_function
        self.routing_type = config.moe_router_load_balancing_type
        if config.moe_router_enable_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(self.num_experts, dtype=torch.float32, device=dev))
            self.register_buffer("local_tokens_per_expert", torch.zeros(self.num_experts, dtype=torch.float32, device=dev),
                                 persistent=False)
        else:
            self.expert_bias = None
        self.fix_router = bool(getattr(config, "fix_router", False))
        self.track_load = bool(getattr(config, "print_expert_load", False) or getattr(config, "enable_expert_placement", False))
        self.register_buffer("expert_load", torch.zeros(self.num_experts, dtype=torch.float32), persistent=False)

    @torch.no_grad()
    def permute_experts(self, old, new):
        """After expert weights moved between slots (``old`` / ``new``: slot -> expert id), reorder the router's rows so
        that output column s again scores the expert stored in slot s.  Replicated state: every rank does the same."""
        old_slot = {e: s for s, e in enumerate(old)}
        idx = torch.tensor([old_slot[e] for e in new], device=self.weight.device)
        self.weight.copy_(self.weight.index_select(0, idx))
        if self.expert_bias is not None:
            self.expert_bias.copy_(self.expert_bias.index_select(0, idx))
            self.local_tokens_per_expert.copy_(self.local_tokens_per_expert.index_select(0, idx))

    def pop_expert_load(self):
        """Tokens per expert accumulated since the last call (device tensor), and reset."""
        out = self.expert_load.clone()
        self.expert_load.zero_()
        return out

    def gating(self, x):
        # --moe-router-dtype: the logits (and everything routing derives from them) in fp32 (default) or fp64
        dt = torch.float64 if getattr(self.config, "moe_router_dtype", None) == "fp64" else torch.float32
        return torch.nn.functional.linear(x.to(dt), self.weight.to(dt))

    def _aux(self, probs_for_loss, routing_map, tokens_per_expert, activation, seq_shape):
        cfg = self.config
        if cfg.moe_aux_loss_coeff <= 0 or not self.training or self.routing_type in ("none", "sinkhorn"):
            return activation
        tp_cp = ps.get_tensor_and_context_parallel_world_size() if cfg.sequence_parallel or ps.get_context_parallel_world_size() > 1 else 1
        coeff = cfg.moe_aux_loss_coeff / max(tp_cp, 1)
        if self.routing_type == "seq_aux_loss":
            s, b = seq_shape
            aux = sequence_load_balancing_loss_func(probs_for_loss, routing_map, b, s, self.topk, coeff)
        else:
            aux = switch_load_balancing_loss_func(probs_for_loss, tokens_per_expert.float(), self.topk, coeff)
        track_moe_metrics(ps.get_moe_layer_wise_logging_tracker(), "load_balancing_loss", aux / max(coeff, 1e-30) * cfg.moe_aux_loss_coeff,
                          self.layer_number, cfg.num_layers)
        return MoEAuxLossAutoScaler.apply(activation, aux)

    def routing(self, logits, seq_shape):
        cfg = self.config
        logits = logits.view(-1, self.num_experts)
        if cfg.moe_z_loss_coeff and self.training:
            logits = MoEAuxLossAutoScaler.apply(logits, z_loss_func(logits, cfg.moe_z_loss_coeff))
        if self.fix_router:
            # deterministic round-robin routing for performance experiments (reference: --fix-router)
            T = logits.shape[0]
            idx = (torch.arange(T, device=logits.device).unsqueeze(1) * self.topk +
                   torch.arange(self.topk, device=logits.device).unsqueeze(0)) % self.num_experts
            probs = torch.zeros_like(logits).scatter(1, idx, 1.0 / self.topk)
            rmap = torch.zeros_like(logits, dtype=torch.int32).scatter(1, idx, 1).bool()
            return probs, rmap
        probs, rmap, tpe = topk_softmax_with_capacity(
            logits, self.topk, cfg.moe_expert_capacity_factor, cfg.moe_pad_expert_input_to_capacity, cfg.moe_token_drop_policy,
            cfg.moe_router_pre_softmax, cfg.moe_router_num_groups, cfg.moe_router_group_topk,
            cfg.moe_router_topk_scaling_factor, self.score_function, self.expert_bias)
        if self.expert_bias is not None and self.training:
            with torch.no_grad():
                self.local_tokens_per_expert += rmap.sum(0).float()
        if self.track_load and self.training:
            # tokens routed to each expert since the last report (--print-expert-load / --enable-expert-placement)
            with torch.no_grad():
                self.expert_load += rmap.sum(0).float()
        if self.score_function == "softmax":
            scores_for_loss = torch.softmax(logits.float(), dim=-1)
        else:
            sg = torch.sigmoid(logits.float())
            scores_for_loss = sg / (sg.sum(-1, keepdim=True) + 1e-20)
        probs = self._aux(scores_for_loss, rmap, tpe, probs, seq_shape)
        return probs, rmap

    def update_expert_bias(self):
        """Aux-loss-free balancing: move each expert's bias against its load (called once per step)."""
        if self.expert_bias is None:
            return
        import torch.distributed as dist
        with torch.no_grad():
            load = self.local_tokens_per_expert.clone()
            if dist.is_initialized():
                g = ps.get_data_parallel_group(with_context_parallel=True)
                if g is not None and dist.get_world_size(g) > 1:
                    dist.all_reduce(load, group=g)
            self.expert_bias += torch.sign(load.mean() - load) * self.config.moe_router_bias_update_rate
            self.local_tokens_per_expert.zero_()

    def forward(self, hidden):
        s, b = hidden.shape[0], hidden.shape[1]
        x = hidden
        if self.config.moe_input_jitter_eps and self.training:
            eps = self.config.moe_input_jitter_eps
            x = x * torch.empty_like(x).uniform_(1 - eps, 1 + eps)
        return self.routing(self.gating(x), (s, b))
