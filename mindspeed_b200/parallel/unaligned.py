"""Tensor / sequence parallel layers for sizes that do not divide by the group size ("unaligned linear").

Dimension ``n`` is split so that the first ``n % world`` ranks get one extra element (for attention: heads, so the
per-rank width is ``heads_r * head_dim``).  Collectives use explicit size lists: all_gather of differently sized
shards, reduce-scatter emulated by all-reduce + slice (reference: mindspeed/core/tensor_parallel/unaligned_layers/
unaligned_utils.py:7-304, unaligned_column_parallel_linear.py:13-250, unaligned_row_parallel_linear.py:12-206).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn

from . import mappings as M
from . import parallel_state as ps


def split_sizes(total: int, world: int, unit: int = 1) -> List[int]:
    """Sizes per rank when ``total`` (a multiple of ``unit``) is split as evenly as possible in multiples of ``unit``."""
    n = total // unit
    base, rem = divmod(n, world)
    return [(base + (1 if r < rem else 0)) * unit for r in range(world)]


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        M.all_reduce(g, ctx.group)
        return g, None


class _GatherLastUneven(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, sizes
        return M.all_gather_uneven(x, group, sizes, x.dim() - 1)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        start = sum(ctx.sizes[:r])
        return g[..., start:start + ctx.sizes[r]].contiguous(), None, None


class UnalignedColumnParallelLinear(nn.Module):
    def __init__(self, input_size, output_size, *, config, init_method, bias=True, gather_output=False, unit=1,
                 sequence_parallel_sizes=None, tp_group=None):
        super().__init__()
        self.group = tp_group if tp_group is not None else ps.get_tensor_model_parallel_group(check_initialized=False)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.sizes = split_sizes(output_size, self.world, unit)
        self.gather_output = gather_output
        self.seq_sizes = sequence_parallel_sizes          # per-rank sequence lengths when the input is sequence sharded
        full = torch.empty(output_size, input_size)
        init_method(full)
        start = sum(self.sizes[:self.rank])
        self.weight = nn.Parameter(full[start:start + self.sizes[self.rank]].clone().to(config.params_dtype))
        self.bias = nn.Parameter(torch.zeros(self.sizes[self.rank], dtype=config.params_dtype)) if bias else None
        self.weight.tensor_model_parallel, self.weight.partition_dim = True, 0

    def forward(self, x):
        if self.seq_sizes is not None and self.world > 1:
            x = M.gather_uneven_first_dim(x, self.group, self.seq_sizes)
        elif self.world > 1:
            x = _CopyToRegion.apply(x, self.group)
        y = torch.nn.functional.linear(x, self.weight, self.bias)
        if self.gather_output and self.world > 1:
            y = _GatherLastUneven.apply(y, self.group, self.sizes)
        return y, None


class UnalignedRowParallelLinear(nn.Module):
    def __init__(self, input_size, output_size, *, config, init_method, bias=True, unit=1, sequence_parallel_sizes=None,
                 tp_group=None):
        super().__init__()
        self.group = tp_group if tp_group is not None else ps.get_tensor_model_parallel_group(check_initialized=False)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.sizes = split_sizes(input_size, self.world, unit)
        self.seq_sizes = sequence_parallel_sizes
        full = torch.empty(output_size, input_size)
        init_method(full)
        start = sum(self.sizes[:self.rank])
        self.weight = nn.Parameter(full[:, start:start + self.sizes[self.rank]].clone().to(config.params_dtype))
        self.bias = nn.Parameter(torch.zeros(output_size, dtype=config.params_dtype)) if bias else None
        self.weight.tensor_model_parallel, self.weight.partition_dim = True, 1

    def forward(self, x):
        y = torch.nn.functional.linear(x, self.weight)
        if self.world > 1:
            if self.seq_sizes is not None:
                y = M.reduce_scatter_uneven_first_dim(y, self.group, self.seq_sizes)
            else:
                y = M.reduce_from_tensor_model_parallel_region(y, self.group)
        if self.bias is not None:
            y = y + self.bias
        return y, None
