"""Norms over a hidden dimension that is itself sharded (2-D tensor parallelism): the statistics are all-reduced over
the group that splits the hidden dimension (reference: mindspeed/core/tensor_parallel/tp_2d/layernorm_2d.py:31-180,
rms_norm_2d.py:30-99)."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import parallel_state as ps


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.clone()
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        if ctx.group is not None and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


def _hidden_group(group):
    if group is not None:
        return group
    return ps.get_tp_y_group() if ps.model_parallel_is_initialized() and "tp_y" in ps._S.groups else None


class RMSNorm2D(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, config=None, group=None):
        super().__init__()
        self.group = _hidden_group(group)
        n = dist.get_world_size(self.group) if self.group is not None else 1
        self.full, self.eps = hidden_size, eps
        dtype = torch.float32 if config is None else config.params_dtype
        self.weight = nn.Parameter(torch.ones(hidden_size // n, dtype=dtype))

    def forward(self, x):
        ss = _AllReduceSum.apply(x.float().pow(2).sum(-1, keepdim=True), self.group)
        return (x.float() * torch.rsqrt(ss / self.full + self.eps) * self.weight.float()).to(x.dtype)


class LayerNorm2D(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, config=None, group=None):
        super().__init__()
        self.group = _hidden_group(group)
        n = dist.get_world_size(self.group) if self.group is not None else 1
        self.full, self.eps = hidden_size, eps
        dtype = torch.float32 if config is None else config.params_dtype
        self.weight = nn.Parameter(torch.ones(hidden_size // n, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size // n, dtype=dtype))

    def forward(self, x):
        xf = x.float()
        mean = _AllReduceSum.apply(xf.sum(-1, keepdim=True), self.group) / self.full
        var = _AllReduceSum.apply((xf - mean).pow(2).sum(-1, keepdim=True), self.group) / self.full
        return ((xf - mean) * torch.rsqrt(var + self.eps) * self.weight.float() + self.bias.float()).to(x.dtype)
