"""Normalisation factory: LayerNorm / RMSNorm, fused or eager
(reference: PTNorm in mindspeed/core/megatron_basic/megatron_basic.py:76-111,
RMSNorm in mindspeed/core/fusions/fused_rms_norm.py:7-42)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.norm import add_rms_norm, rms_norm


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, config=None, sequence_parallel=False):
        super().__init__()
        dev = None if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        dtype = torch.float32 if config is None else config.params_dtype
        zero_centered = bool(config is not None and config.layernorm_zero_centered_gamma)
        init = torch.zeros if zero_centered else torch.ones
        self.weight = nn.Parameter(init(hidden_size, device=dev, dtype=dtype))
        self.eps, self.zero_centered = eps, zero_centered
        self.fused = bool(config is not None and (config.use_fused_rmsnorm or config.optimization_level >= 1))
        setattr(self.weight, "sequence_parallel", sequence_parallel)

    def forward(self, x):
        return rms_norm(x, self.weight, self.eps, self.zero_centered, fused=self.fused)

    def forward_add(self, x, residual):
        """(x + residual, norm(x + residual)): the residual add rides in the norm's pass over the row."""
        return add_rms_norm(x, residual, self.weight, self.eps, self.zero_centered, fused=self.fused)


class LayerNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, config=None, sequence_parallel=False):
        super().__init__()
        dev = None if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        dtype = torch.float32 if config is None else config.params_dtype
        self.weight = nn.Parameter(torch.ones(hidden_size, device=dev, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size, device=dev, dtype=dtype))
        self.eps, self.hidden_size = eps, hidden_size
        setattr(self.weight, "sequence_parallel", sequence_parallel)
        setattr(self.bias, "sequence_parallel", sequence_parallel)

    def forward(self, x):
        return F.layer_norm(x, (self.hidden_size,), self.weight, self.bias, self.eps)


class IdentityOp(nn.Module):
    def forward(self, x, *a, **k):
        return x


def build_norm(config, hidden_size, eps=None):
    """``PTNorm``-style factory keyed on ``config.normalization``."""
    eps = config.layernorm_epsilon if eps is None else eps
    if config.normalization == "RMSNorm":
        if getattr(config, "tp_2d", False):
            from ..parallel.tp2d.norm_2d import RMSNorm2D
            return RMSNorm2D(hidden_size, eps, config)
        return RMSNorm(hidden_size, eps, config, sequence_parallel=config.sequence_parallel)
    if config.normalization == "LayerNorm":
        if getattr(config, "tp_2d", False):
            from ..parallel.tp2d.norm_2d import LayerNorm2D
            return LayerNorm2D(hidden_size, eps, config)
        return LayerNorm(hidden_size, eps, config, sequence_parallel=config.sequence_parallel)
    raise ValueError(f"unknown normalization {config.normalization}")


PTNorm = build_norm
