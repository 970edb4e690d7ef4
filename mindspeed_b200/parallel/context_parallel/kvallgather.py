"""KV-allgather context parallelism (Llama-3 style): all-gather K and V once, then each rank attends its two
load-balanced query chunks to the key prefix they may see
(reference: mindspeed/te/pytorch/attention/dot_product_attention/kvallgather_context_parallel.py:119-400; causal only).
The gather is differentiable (reduce-scatter of dK/dV in backward)."""
from __future__ import annotations

import torch

from ...ops import attention as A
from .. import mappings as M
from .. import parallel_state as ps


def kv_allgather_attention(q, k, v, config=None, softmax_scale=None):
    group = ps.get_context_parallel_group()
    cp, r = ps.get_context_parallel_world_size(), ps.get_context_parallel_rank()
    s_local = q.shape[0]
    c = s_local // 2
    # gathered layout is rank-major [cp, 2 chunks]: reorder to sequence order of the 2cp chunks
    kg = M.gather_from_sequence_parallel_region(k, tensor_parallel_output_grad=True, group=group)
    vg = M.gather_from_sequence_parallel_region(v, tensor_parallel_output_grad=True, group=group)
    order = [0] * (2 * cp)
    for j in range(cp):
        order[j] = 2 * j
        order[2 * cp - 1 - j] = 2 * j + 1
    idx = torch.tensor(order, device=q.device)
    kg = kg.reshape(2 * cp, c, *k.shape[1:]).index_select(0, idx).reshape(2 * cp * c, *k.shape[1:])
    vg = vg.reshape(2 * cp, c, *v.shape[1:]).index_select(0, idx).reshape(2 * cp * c, *v.shape[1:])
    outs = []
    for qi, chunk in ((0, r), (1, 2 * cp - 1 - r)):
        qc = q[qi * c:(qi + 1) * c]
        kd, vd = kg[chunk * c:(chunk + 1) * c], vg[chunk * c:(chunk + 1) * c]
        if chunk > 0:
            outs.append(_PrefixCausalAttn.apply(qc, kg[:chunk * c], vg[:chunk * c], kd, vd, softmax_scale))
        else:
            outs.append(_PrefixCausalAttn.apply(qc, None, None, kd, vd, softmax_scale))
    return torch.cat(outs, dim=0)


class _PrefixCausalAttn(torch.autograd.Function):
    """Attention of one query chunk to [key prefix (no mask) | own key chunk (causal)], computed as two blocks merged
    by log-sum-exp.  Backward differentiates each block with the GLOBAL output and LSE, which is exact."""

    @staticmethod
    def forward(ctx, q, kp, vp, kd, vd, scale):
        q, kd, vd = q.contiguous(), kd.contiguous(), vd.contiguous()
        o, l, c2 = A.attn_fwd_block(q, kd, vd, True, scale)
        c1 = None
        if kp is not None:
            kp, vp = kp.contiguous(), vp.contiguous()
            o1, l1, c1 = A.attn_fwd_block(q, kp, vp, False, scale)
            o, l = A.merge_lse(o1, l1, o, l)
        o, l = o.contiguous(), l.contiguous()
        ctx.has_prefix = kp is not None
        ctx.save_for_backward(q, kd, vd, o, l, *((kp, vp) if kp is not None else ()))
        ctx.meta = (scale, c1, c2)
        return o

    @staticmethod
    def backward(ctx, do):
        scale, c1, c2 = ctx.meta
        saved = ctx.saved_tensors
        q, kd, vd, o, l = saved[:5]
        do = do.contiguous()
        dq, dkd, dvd = A.attn_bwd_block(do, q, kd, vd, o, l, True, scale, c2)
        dkp = dvp = None
        if ctx.has_prefix:
            kp, vp = saved[5], saved[6]
            dq1, dkp, dvp = A.attn_bwd_block(do, q, kp, vp, o, l, False, scale, c1)
            dq = dq + dq1
        return dq, dkp, dvp, dkd, dvd, None
