"""Expert MLPs.

``GroupedMLP`` keeps the local experts' weights stacked ([E_local, hidden, 2*ffn] and [E_local, ffn, hidden]) and runs a
grouped GEMM over expert-sorted tokens: y[rows of expert e] = x[rows of expert e] @ W[e].  On a GPU the per-expert
products run on the tcgen05 GEMM kernel (``ops.grouped_gemm``); the activation is the (probability-weighted) SwiGLU
kernel.  reference: mindspeed/core/transformer/moe/grouped_matmul_util.py:138-397, mindspeed/ops/gmm.py:20-175.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...models.mlp import MLP
from ...ops.activation import swiglu
from ...ops.grouped_gemm import grouped_gemm
from .. import parallel_state as ps


class GroupedMLP(nn.Module):
    def __init__(self, num_local_experts, config):
        super().__init__()
        self.config, self.num_local_experts = config, num_local_experts
        etp = ps.get_expert_tensor_parallel_world_size()
        ffn = config.moe_ffn_hidden_size // etp
        self.ffn = ffn
        fc1_out = 2 * ffn if config.gated_linear_unit else ffn
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight1 = nn.Parameter(torch.empty(num_local_experts, config.hidden_size, fc1_out, device=dev, dtype=config.params_dtype))
        self.weight2 = nn.Parameter(torch.empty(num_local_experts, ffn, config.hidden_size, device=dev, dtype=config.params_dtype))
        if config.perform_initialization:
            from ..random import get_cuda_rng_tracker, get_expert_parallel_rng_tracker_name
            tr = get_cuda_rng_tracker()
            def init():
                with torch.no_grad():
                    for e in range(num_local_experts):
                        w1 = torch.empty(fc1_out, config.hidden_size, device=self.weight1.device, dtype=torch.float32)
                        config.init_method(w1)
                        self.weight1[e].copy_(w1.t())
                        w2 = torch.empty(config.hidden_size, ffn, device=self.weight2.device, dtype=torch.float32)
                        config.output_layer_init_method(w2)
                        self.weight2[e].copy_(w2.t())
            if tr.is_initialized() and self.weight1.is_cuda:
                with tr.fork(get_expert_parallel_rng_tracker_name()):
                    init()
            else:
                init()
        for w in (self.weight1, self.weight2):
            setattr(w, "allreduce", False)
        self.fused = config.optimization_level >= 1

    def forward(self, permuted_tokens, tokens_per_expert, permuted_probs=None):
        """permuted_tokens [R, H] sorted by local expert; tokens_per_expert [E_local] (host list or tensor)."""
        return self.run(permuted_tokens, tokens_per_expert, permuted_probs, self.weight1, self.weight2), None

    def run(self, permuted_tokens, tokens_per_expert, permuted_probs, weight1, weight2):
        """The expert MLP on explicit stacked weights [n, H, F1] / [n, F, H] (the module's own, or replicas of other
        ranks' experts)."""
        if permuted_tokens.shape[0] == 0:
            # keep the parameters in the graph so data-parallel reduction sees zero gradients, and the probabilities too:
            # their all-to-all has a backward collective that the peers run, so this rank must run it as well
            z = (weight1.sum() + weight2.sum()) * 0
            if permuted_probs is not None:
                z = z + permuted_probs.sum().to(z.dtype) * 0
            return permuted_tokens + z.to(permuted_tokens.dtype)
        h = grouped_gemm(permuted_tokens, weight1, tokens_per_expert, trans_b=False)
        if self.config.gated_linear_unit and self.config.activation_func is F.silu:
            a = swiglu(h, permuted_probs, fused=self.fused)
        else:
            if self.config.gated_linear_unit:
                g, u = h.chunk(2, dim=-1)
                a = self.config.activation_func(g) * u
            else:
                a = self.config.activation_func(h)
            if permuted_probs is not None:
                a = a * permuted_probs.unsqueeze(-1).to(a.dtype)
        return grouped_gemm(a, weight2, tokens_per_expert, trans_b=False)


class SequentialMLP(nn.Module):
    def __init__(self, num_local_experts, config):
        super().__init__()
        self.config, self.num_local_experts = config, num_local_experts
        self.local_experts = nn.ModuleList([MLP(config, ffn_hidden_size=config.moe_ffn_hidden_size, is_expert=True)
                                            for _ in range(num_local_experts)])

    def forward(self, permuted_tokens, tokens_per_expert, permuted_probs=None):
        sizes = tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)
        outs = []
        pp = torch.split(permuted_probs, sizes) if permuted_probs is not None else [None] * len(sizes)
        for e, (x, pr) in enumerate(zip(torch.split(permuted_tokens, sizes), pp)):
            y, _ = self.local_experts[e](x)
            if pr is not None:
                y = y * pr.unsqueeze(-1).to(y.dtype)
            outs.append(y)
        return torch.cat(outs, dim=0), None


class SharedExpertMLP(MLP):
    """Always-on expert(s) added to the routed output; can run on a side stream to overlap the dispatch all-to-all
    (reference: shared-expert overlap in mindspeed/core/transformer/moe/moe_feature/overlap/token_dispatcher.py:797-808)."""

    def __init__(self, config):
        super().__init__(config, ffn_hidden_size=config.moe_shared_expert_intermediate_size)
        self.stream = None

    def forward(self, hidden_states):
        out, _ = super().forward(hidden_states)
        return out
