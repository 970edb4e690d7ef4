"""The DeepSpeed-style MoE as the MLP of a transformer layer (``--moe-model-type deepspeed_moe``).

``LegacyMoEBlock(config)`` has the call shape of the framework's MoE layer (``forward(hidden) -> (output, bias)``) and builds
a ``MoE`` from the training flags: top-1 / top-2 gating with capacity (``--moe-train-capacity-factor``, ``--moe-no-drop`` lifts
the capacity to "every token fits"), optional noisy gating (``--noisy-gate-policy``), experts split over the expert-parallel
group, and the capacity dimension cut into ``--pipe-experts-multi-data`` chunks whose all-to-alls and expert computations
alternate (``--use-pipe-experts``; with ``--pipe-experts-multi-stream`` the chunks' all-to-alls run on a second stream so that
chunk i + 1 is exchanged while chunk i computes).  The load-balancing loss of the gate enters the graph through the same
auxiliary-loss hook the core router uses, scaled by ``--moe-aux-loss-coeff``.
reference: mindspeed/moe/{moe,mixtral_parallel_mlpbm,pipe_experts}.py and the flags of mindspeed/arguments.py:119-170.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel import parallel_state as ps
from .layer import MoE


class LegacyMoEBlock(nn.Module):
    def __init__(self, config, layer_number: int = 1):
        super().__init__()
        from ..models.mlp import MLP
        self.config = config
        ep = ps.get_expert_model_parallel_world_size()
        k = int(getattr(config, "moe_router_topk", 2) or 2)
        if k not in (1, 2):
            raise ValueError("the DeepSpeed-style gate supports top-1 and top-2 routing")
        cf = float(getattr(config, "moe_train_capacity_factor", 1.0) or 1.0)
        if getattr(config, "moe_no_drop", False):
            cf = float(config.num_moe_experts)          # capacity = all tokens: nothing is dropped
        pipe = int(getattr(config, "pipe_experts_multi_data", 1) or 1) if getattr(config, "use_pipe_experts", False) else 1
        ffn = getattr(config, "moe_ffn_hidden_size", None) or config.ffn_hidden_size

        def expert():
            return MLP(config, ffn_hidden_size=ffn, is_expert=True)
        self.moe = MoE(config.hidden_size, expert, num_experts=config.num_moe_experts, ep_size=ep, k=k, capacity_factor=cf,
                       eval_capacity_factor=cf, noisy_gate_policy=getattr(config, "noisy_gate_policy", None),
                       ep_group=ps.get_expert_model_parallel_group(check_initialized=False) if ep > 1 else None, pipe_experts=pipe,
                       use_rts=bool(getattr(config, "use_rts", False)))
        self.moe.moe_layer.multi_stream = bool(getattr(config, "pipe_experts_multi_stream", False))
        self.aux_coeff = float(getattr(config, "moe_aux_loss_coeff", 0.0) or 0.0)

    def forward(self, hidden_states):
        from ..parallel.moe.moe_utils import MoEAuxLossAutoScaler
        out, l_aux, _ = self.moe(hidden_states)
        if self.training and self.aux_coeff > 0 and l_aux is not None:
            out = MoEAuxLossAutoScaler.apply(out, l_aux * self.aux_coeff)
        return out, None
