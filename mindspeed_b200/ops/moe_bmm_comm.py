"""MoE batch-matmul ops with their expert-parallel / tensor-parallel collectives (the ``--moe-bmm-mc2`` pair) and the
grouped-matmul + all-reduce op.

Data layout of the pair (E experts in total, ep x tp ranks; this rank holds E/ep experts and 1/tp of every expert's
hidden width):

  all_to_all_all_gather_bmm(x [E, C, H/tp?], w [E/ep, H, M/tp])
        tokens bucketed per *global* expert go to the rank group that owns the expert (all-to-all over ep, dim 0), the
        tensor-parallel shards of each bucket are all-gathered (over tp, along ``shard`` = tokens (1) or hidden (0)) and
        multiplied by the local experts' weights: y [E/ep, ep*C (*tp), M/tp]
  bmm_reduce_scatter_all_to_all(x [E/ep, ep*C (*tp), M/tp], w [E/ep, M/tp, H])
        the mirror: batch matmul, reduce-scatter over tp (partial sums of the M/tp contraction), all-to-all back over ep.
  grouped_matmul_all_reduce(x, weights, group_list, group)
        per-group matmul of row segments followed by one all-reduce (row-parallel grouped linear).

The collectives are the autograd-aware mappings, so the pair is differentiable; on a GPU the batch matmul goes through
the tcgen05 grouped GEMM.  reference: mindspeed/ops/npu_all_to_all_all_gather_bmm.py, npu_bmm_reduce_scatter_all_to_all.py,
npu_grouped_mat_mul_all_reduce.py; users: mindspeed/core/transformer/moe/grouped_gemm_util.py:57-228.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..parallel import mappings as M
from .grouped_gemm import grouped_gemm

_ACT = {None: lambda t: t, "none": lambda t: t, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu,
        "relu": torch.nn.functional.relu, "fastgelu": lambda t: t * torch.sigmoid(1.702 * t)}


def _bmm(x, w):
    """x [G, R, K] @ w [G, K, N]; grouped GEMM on the GPU path, torch.bmm otherwise."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        G, R, K = x.shape
        return grouped_gemm(x.reshape(G * R, K), w, [R] * G, trans_b=False).view(G, R, w.shape[-1])
    return torch.bmm(x, w)


def all_to_all_all_gather_bmm(x, weight, group_ep, group_tp, bias=None, shard_type: int = 1, act_type: Optional[str] = None,
                              need_allgather_out: bool = False, need_activation_feature: bool = False):
    """x [E, C, H]; weight [E/ep, H, M/tp].  shard_type 1: the tp ranks hold different tokens (gather along C);
    shard_type 0: they hold different slices of H (gather along H)."""
    ep = M._ws(group_ep)
    E, C, H = x.shape
    e_loc = E // ep
    if ep > 1:
        # send bucket (e) to rank e // e_loc: rows of dim 0 are already grouped by destination
        recv = M.all_to_all(group_ep, x.contiguous())                          # [ep * e_loc, C, H], source-major
        recv = recv.view(ep, e_loc, C, H).permute(1, 0, 2, 3).reshape(e_loc, ep * C, H)
    else:
        recv = x
    if M._ws(group_tp) > 1:
        if shard_type == 1:
            g = M.gather_from_sequence_parallel_region(recv.transpose(0, 1).contiguous(), True, group_tp)
            gathered = g.transpose(0, 1).contiguous()                            # tokens of all tp ranks
        else:
            gathered = M.gather_from_tensor_model_parallel_region(recv, group_tp)
    else:
        gathered = recv
    y = _bmm(gathered, weight)
    if bias is not None:
        y = y + bias
    pre = y
    y = _ACT[act_type](y)
    outs = [y]
    if need_allgather_out:
        outs.append(gathered)
    if need_activation_feature:
        outs.append(pre)
    return outs[0] if len(outs) == 1 else tuple(outs)


def bmm_reduce_scatter_all_to_all(x, weight, group_ep, group_tp, bias=None, shard_type: int = 1):
    """x [E/ep, R, M/tp]; weight [E/ep, M/tp, H] -> [E, C, H] back on the token owners."""
    ep = M._ws(group_ep)
    y = _bmm(x, weight)                                                        # partial over the M/tp contraction
    if M._ws(group_tp) > 1:
        if shard_type == 1:
            y = M.reduce_scatter_to_sequence_parallel_region(y.transpose(0, 1).contiguous(), group_tp).transpose(0, 1).contiguous()
        else:
            y = M.reduce_from_tensor_model_parallel_region(y, group_tp)
            y = M.scatter_to_tensor_model_parallel_region(y, group_tp)
    e_loc, R, H = y.shape
    if ep > 1:
        C = R // ep
        send = y.view(e_loc, ep, C, H).permute(1, 0, 2, 3).reshape(ep * e_loc, C, H).contiguous()
        y = M.all_to_all(group_ep, send)                                       # [E, C, H]
    if bias is not None:
        y = y + bias
    return y


def grouped_matmul_all_reduce(x: torch.Tensor, weights: Sequence[torch.Tensor], group_list: Sequence[int], group,
                              bias: Optional[Sequence[torch.Tensor]] = None) -> torch.Tensor:
    """x [R, K_local] with rows split by ``group_list`` (sizes); weights[g] [K_local, N]; sum over the group's ranks."""
    outs, s = [], 0
    for g, n in enumerate(group_list):
        seg = x[s:s + n]
        o = seg @ weights[g]
        if bias is not None and bias[g] is not None and M._rk(group) == 0:
            o = o + bias[g]
        outs.append(o)
        s += n
    y = torch.cat(outs, dim=0) if outs else x.new_zeros(0, weights[0].shape[-1])
    return M.reduce_from_tensor_model_parallel_region(y, group)
