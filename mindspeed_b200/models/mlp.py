"""Dense MLP: column-parallel FC1 -> activation (GeLU / SwiGLU) -> row-parallel FC2."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.activation import swiglu
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, linear_classes
from ..parallel.random import CheckpointWithoutOutput


class MLP(nn.Module):
    def __init__(self, config, ffn_hidden_size=None, is_expert=False, input_size=None):
        super().__init__()
        self.config = config
        ffn = ffn_hidden_size or config.ffn_hidden_size
        inp = input_size or config.hidden_size
        fc1_out = ffn * 2 if config.gated_linear_unit else ffn
        Col, Row = linear_classes(config)
        self.linear_fc1 = Col(inp, fc1_out, config=config, init_method=config.init_method,
                                               bias=config.add_bias_linear, skip_bias_add=True, is_expert=is_expert,
                                               stride=2 if config.gated_linear_unit else 1)
        self.linear_fc2 = Row(ffn, config.hidden_size, config=config,
                                            init_method=config.output_layer_init_method, bias=config.add_bias_linear,
                                            input_is_parallel=True, skip_bias_add=True, is_expert=is_expert)
        self.activation_func = config.activation_func
        self.fused_swiglu = config.use_fused_swiglu or config.optimization_level >= 1
        # "activation-function recompute": drop the activation output, rebuild it before FC2's backward
        # (reference: mindspeed/core/memory/recompute/activation/*, --recompute-activation-function)
        self.recompute_activation = bool(getattr(config, "recompute_activation_function", False))

    def _act(self, h, bias):
        if bias is not None:
            h = h + bias
        if self.config.gated_linear_unit:
            if self.activation_func is F.silu:
                return swiglu(h, fused=self.fused_swiglu)
            a, b = h.chunk(2, dim=-1)
            return self.activation_func(a) * b
        return self.activation_func(h)

    def forward(self, hidden_states):
        level = getattr(self.config, "compress_dense", "disable")
        if level in ("level0", "level1") and self.training and torch.is_grad_enabled() and not getattr(self, "is_expert", False):
            # --compress-dense: level0 stores the MLP's input compressed, level1 everything the MLP saves for backward
            from ..memory.compress_activation import CompressSavedActivations
            only = {hidden_states.data_ptr()} if level == "level0" else None
            with CompressSavedActivations(only=only):
                return self._forward(hidden_states)
        return self._forward(hidden_states)

    def _forward(self, hidden_states):
        h, b1 = self.linear_fc1(hidden_states)
        if self.recompute_activation and self.training and h.requires_grad:
            ck = CheckpointWithoutOutput()
            a = ck.checkpoint(lambda t: self._act(t, b1), False, h)
            out, b2 = self.linear_fc2(a)
            ck.discard_output()
            out.register_hook(ck.recompute)
        else:
            out, b2 = self.linear_fc2(self._act(h, b1))
        return out, b2
