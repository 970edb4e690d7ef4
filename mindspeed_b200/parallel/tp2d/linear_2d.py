"""2-D tensor parallel linear: the weight is sharded along both of its dimensions.

Activation layout [s/(a*cp), b, h/r]: sequence split over the all-gather group (size a), hidden split over the
reduce-scatter group (size r).  One linear is
     all-gather over the ag group (sequence) -> GEMM with W[out/a, in/r]^T -> reduce-scatter over the rs group (sequence)
giving [s/(r*cp), b, out/a]; the next linear swaps the two groups, so activations never exist unsharded.
Overlap modes of the reference (ring-P2P all-gather || GEMM, chunked GEMM || reduce-scatter, fused kernel:
mindspeed/core/tensor_parallel/tp_2d/linear_2d_split_along_first_dim.py:102-126,266-357) map onto the comm_ops
back ends here: the all-gather->GEMM half and the GEMM->reduce-scatter half are the same fused kernels the 1-D
layers use, each on its own group.  reference module: tp_2d/parallel_linear_2d.py:24-207.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import mappings as M
from .. import parallel_state as ps
from ..comm_ops import get_ops


class _Linear2DFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ag_group, rs_group):
        ops = get_ops()
        ctx.groups = (ag_group, rs_group)
        ctx.save_for_backward(x, w)
        total = M.all_gather_first_dim(x, ag_group)
        return ops.matmul_reduce_scatter(total, w, rs_group, nt=True)

    @staticmethod
    def backward(ctx, dy):
        ops = get_ops()
        ag_group, rs_group = ctx.groups
        x, w = ctx.saved_tensors
        # adjoint: all-gather dY over the rs group, dX_total = dY_total @ W, reduce-scatter over the ag group
        dx, dy_total = ops.allgather_matmul(dy.contiguous(), w, rs_group, nt=False, need_gathered=True)
        dx = M.reduce_scatter_first_dim(dx, ag_group)
        total = M.all_gather_first_dim(x, ag_group)
        dw = ops.wgrad(dy_total, total, None).to(w.dtype)
        return dx, dw, None, None


class ParallelLinear2D(nn.Module):
    def __init__(self, input_size, output_size, *, config, init_method, ag_group, rs_group, bias=False):
        super().__init__()
        self.ag_group, self.rs_group = ag_group, rs_group
        a = dist.get_world_size(ag_group) if ag_group is not None else 1
        r = dist.get_world_size(rs_group) if rs_group is not None else 1
        ai = dist.get_rank(ag_group) if ag_group is not None else 0
        ri = dist.get_rank(rs_group) if rs_group is not None else 0
        if output_size % a or input_size % r:
            raise ValueError("2-D tensor parallel linear: sizes must divide by the group sizes")
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.empty(output_size // a, input_size // r, device=dev, dtype=config.params_dtype))
        if config.perform_initialization:
            full = torch.empty(output_size, input_size)
            init_method(full)
            with torch.no_grad():
                self.weight.copy_(full.chunk(a, 0)[ai].chunk(r, 1)[ri])
        self.bias = nn.Parameter(torch.zeros(output_size // a, device=dev, dtype=config.params_dtype)) if bias else None

    def forward(self, x):
        y = _Linear2DFn.apply(x, self.weight, self.ag_group, self.rs_group)
        if self.bias is not None:
            y = y + self.bias
        return y, None
