"""Autograd-aware collectives between tensor-/sequence-/expert-parallel regions.

Function names follow Megatron-core ``tensor_parallel.mappings``.  Each forward
collective is paired with its adjoint in backward:

  copy      : identity            / all-reduce
  reduce    : all-reduce          / identity
  scatter   : split last dim      / all-gather last dim
  gather    : all-gather last dim / split last dim
  SP scatter: split first dim     / all-gather first dim
  SP gather : all-gather first dim/ reduce-scatter (or split) first dim
  SP reduce-scatter               / all-gather first dim
  all-to-all (optionally with split sizes) is self-adjoint with sizes swapped.

Works on NCCL (GPU) and gloo (CPU) groups; gloo lacks reduce_scatter_tensor, which is
emulated with all_reduce + slice so that the CPU tests cover the same call graph.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import parallel_state as ps


def _ws(group):
    return 1 if group is None else dist.get_world_size(group)


def _rk(group):
    return 0 if group is None else dist.get_rank(group)


def _is_gloo(group) -> bool:
    try:
        return dist.get_backend(group) == "gloo"
    except Exception:
        return False


# ---- raw collectives -------------------------------------------------------------------
def all_reduce(x: torch.Tensor, group, async_op=False):
    if _ws(group) == 1:
        return None
    return dist.all_reduce(x, group=group, async_op=async_op)


def all_gather_first_dim(x: torch.Tensor, group, out: Optional[torch.Tensor] = None, async_op=False):
    n = _ws(group)
    if n == 1:
        return (x, None) if async_op else x
    shape = list(x.shape)
    shape[0] *= n
    if out is None:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    h = dist.all_gather_into_tensor(out, x.contiguous(), group=group, async_op=async_op)
    return (out, h) if async_op else out


def reduce_scatter_first_dim(x: torch.Tensor, group, async_op=False):
    n = _ws(group)
    if n == 1:
        return (x, None) if async_op else x
    if x.shape[0] % n != 0:
        raise ValueError("first dimension must be divisible by the group size")
    shape = list(x.shape)
    shape[0] //= n
    if _is_gloo(group):
        tmp = x.contiguous().clone()
        dist.all_reduce(tmp, group=group)
        out = tmp[_rk(group) * shape[0]:(_rk(group) + 1) * shape[0]].clone()
        return (out, None) if async_op else out
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    h = dist.reduce_scatter_tensor(out, x.contiguous(), group=group, async_op=async_op)
    return (out, h) if async_op else out


def split_first_dim(x, group):
    n = _ws(group)
    if n == 1:
        return x
    per = x.shape[0] // n
    r = _rk(group)
    return x[r * per:(r + 1) * per].contiguous()


def split_last_dim(x, group):
    n = _ws(group)
    if n == 1:
        return x
    per = x.shape[-1] // n
    r = _rk(group)
    return x[..., r * per:(r + 1) * per].contiguous()


def all_gather_last_dim(x, group):
    n = _ws(group)
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=-1).contiguous()


def all_to_all_single(x, group, output_split_sizes=None, input_split_sizes=None, async_op=False):
    n = _ws(group)
    if n == 1:
        return (x, None) if async_op else x
    x = x.contiguous()
    if output_split_sizes is None:
        out = torch.empty_like(x)
    else:
        out = x.new_empty([sum(output_split_sizes)] + list(x.shape[1:]))
    if _is_gloo(group):
        # gloo has no all-to-all: exchange pairwise with non-blocking send / receive
        ins = list(x.split(input_split_sizes if input_split_sizes is not None else x.shape[0] // n, dim=0))
        outs = list(out.split(output_split_sizes if output_split_sizes is not None else out.shape[0] // n, dim=0))
        me = _rk(group)
        recv_bufs = [torch.empty_like(o) for o in outs]
        reqs = []
        for p in range(n):
            if p == me:
                recv_bufs[p].copy_(ins[p])
                continue
            peer = dist.get_global_rank(group, p)
            if ins[p].numel() > 0:
                reqs.append(dist.isend(ins[p].contiguous(), peer, group=group))
            if recv_bufs[p].numel() > 0:
                reqs.append(dist.irecv(recv_bufs[p], peer, group=group))
        for r in reqs:
            r.wait()
        out = torch.cat(recv_bufs, dim=0)
        return (out, None) if async_op else out
    h = dist.all_to_all_single(out, x, output_split_sizes=output_split_sizes, input_split_sizes=input_split_sizes,
                               group=group, async_op=async_op)
    return (out, h) if async_op else out


# ---- autograd functions ----------------------------------------------------------------
class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        all_reduce(g, ctx.group)
        return g, None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        all_reduce(x, group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_last_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_last_dim(g, ctx.group), None


class _GatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_last_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return split_last_dim(g, ctx.group), None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_first_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_first_dim(g, ctx.group), None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, tensor_parallel_output_grad):
        ctx.group, ctx.tp_grad = group, tensor_parallel_output_grad
        return all_gather_first_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.tp_grad:
            return reduce_scatter_first_dim(g, ctx.group), None, None
        return split_first_dim(g, ctx.group), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_first_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_first_dim(g, ctx.group), None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, output_split_sizes, input_split_sizes):
        ctx.group, ctx.o, ctx.i = group, output_split_sizes, input_split_sizes
        return all_to_all_single(x, group, output_split_sizes, input_split_sizes)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_single(g, ctx.group, ctx.i, ctx.o), None, None, None


def _tp(group):
    return ps.get_tensor_model_parallel_group(check_initialized=False) if group is None else group


def copy_to_tensor_model_parallel_region(x, group=None):
    return _Copy.apply(x, _tp(group))


def reduce_from_tensor_model_parallel_region(x, group=None):
    return _Reduce.apply(x, _tp(group))


def scatter_to_tensor_model_parallel_region(x, group=None):
    return _ScatterLast.apply(x, _tp(group))


def gather_from_tensor_model_parallel_region(x, group=None):
    return _GatherLast.apply(x, _tp(group))


def scatter_to_sequence_parallel_region(x, group=None):
    return _ScatterSeq.apply(x, _tp(group))


def gather_from_sequence_parallel_region(x, tensor_parallel_output_grad=True, group=None, output_split_sizes=None,
                                         use_global_buffer=False):
    if output_split_sizes is not None:
        return gather_uneven_first_dim(x, _tp(group), output_split_sizes)
    return _GatherSeq.apply(x, _tp(group), tensor_parallel_output_grad)


def reduce_scatter_to_sequence_parallel_region(x, group=None, input_split_sizes=None, use_global_buffer=False):
    if input_split_sizes is not None:
        return reduce_scatter_uneven_first_dim(x, _tp(group), input_split_sizes)
    return _ReduceScatterSeq.apply(x, _tp(group))


def all_to_all(group, x, output_split_sizes=None, input_split_sizes=None):
    return _AllToAll.apply(x, group, output_split_sizes, input_split_sizes)


# ---- uneven variants (unaligned TP / MoE with TP) -----------------------------------------
def all_gather_uneven(x, group, sizes: List[int], dim: int = 0):
    """All-gather of shards whose extent along ``dim`` differs per rank: pad to the largest, gather, trim."""
    mx = max(sizes)
    x = x.contiguous()
    if x.shape[dim] < mx:
        pad_shape = list(x.shape)
        pad_shape[dim] = mx - x.shape[dim]
        x = torch.cat((x, x.new_zeros(pad_shape)), dim=dim)
    parts = [torch.empty_like(x) for _ in sizes]
    dist.all_gather(parts, x, group=group)
    return torch.cat([p.narrow(dim, 0, s) for p, s in zip(parts, sizes)], dim=dim)



class _GatherUneven(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, list(sizes)
        return all_gather_uneven(x, group, sizes, 0)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_uneven(g, ctx.group, ctx.sizes), None, None


def _reduce_scatter_uneven(x, group, sizes):
    x = x.contiguous().clone()
    dist.all_reduce(x, group=group)
    r = _rk(group)
    start = sum(sizes[:r])
    return x[start:start + sizes[r]].contiguous()


class _ReduceScatterUneven(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, list(sizes)
        return _reduce_scatter_uneven(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        return all_gather_uneven(g, ctx.group, ctx.sizes, 0), None, None


def gather_uneven_first_dim(x, group, sizes: List[int]):
    if _ws(group) == 1:
        return x
    return _GatherUneven.apply(x, group, sizes)


def reduce_scatter_uneven_first_dim(x, group, sizes: List[int]):
    if _ws(group) == 1:
        return x
    return _ReduceScatterUneven.apply(x, group, sizes)
