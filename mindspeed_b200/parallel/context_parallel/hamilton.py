"""Hamilton attention: ring attention whose KV block travels on several edge-disjoint cycles at once.

Plain ring attention moves a rank's whole KV block to ONE neighbour per step, so of the n-1 links a rank has through
the switch it drives one.  Here the local KV block is cut into ``path_num`` chunks along the sequence and chunk p is sent
around its own Hamiltonian cycle of the rank graph: the cycle with stride ``s_p`` (rank r -> r + s_p mod n), which visits
every rank exactly once when gcd(s_p, n) = 1; cycles with different strides share no directed edge.  Every step a rank
therefore sends to and receives from ``path_num`` different peers, each moving 1/path_num of the block, and after n-1
steps it has attended to every chunk of every rank.  The chunk on path p at step t originated on rank r - t*s_p.

Only full (non-causal) attention: the pieces a rank holds at one step come from different source ranks, so there is no
single triangular mask for the step (same restriction as the reference).  Partial results are merged in log-sum-exp
form; backward runs the same cycles again with dK / dV travelling beside their chunk and one extra hop to bring them home.

reference: HamiltonCPStrategy, mindspeed/te/pytorch/attention/dot_product_attention/context_parallel.py:178-269, and the
list-based all-to-all exchange of hamilton_context_parallel.py:482-502.  On NVSwitch every peer is one hop away, so the
strides need no knowledge of the physical topology.
"""
from __future__ import annotations

import math
from typing import List

import torch
import torch.distributed as dist

from ...ops import attention as A
from .. import parallel_state as ps


def hamilton_strides(n: int, path_num: int) -> List[int]:
    """Strides of the first ``path_num`` edge-disjoint directed Hamiltonian cycles of n ranks (all strides coprime to n)."""
    strides = [s for s in range(1, n) if math.gcd(s, n) == 1]
    if path_num < 1 or path_num > len(strides):
        raise ValueError(f"{n} ranks have {len(strides)} edge-disjoint stride cycles; path_num={path_num} is out of range")
    return strides[:path_num]


def max_paths(n: int) -> int:
    return sum(1 for s in range(1, n) if math.gcd(s, n) == 1)


def _exchange(pieces: List[torch.Tensor], strides: List[int], ranks: List[int], me: int, group, reverse=False):
    """Piece p goes to rank me + s_p and is replaced by the piece from rank me - s_p (the other way round if ``reverse``)."""
    n = len(ranks)
    ops, recv = [], []
    for p, s in enumerate(strides):
        step = -s if reverse else s
        buf = torch.empty_like(pieces[p])
        recv.append(buf)
        ops.append(dist.P2POp(dist.isend, pieces[p].contiguous(), ranks[(me + step) % n], group))
        ops.append(dist.P2POp(dist.irecv, buf, ranks[(me - step) % n], group))
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    return recv


class _HamiltonAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, ranks, path_num, softmax_scale):
        n = len(ranks)
        me = ranks.index(dist.get_rank())
        strides = hamilton_strides(n, path_num)
        if k.shape[0] % path_num != 0:
            raise ValueError(f"local KV length {k.shape[0]} is not divisible by path_num={path_num}")
        out, lse, _ = A.attn_fwd_block(q, k, v, False, softmax_scale)
        lse = lse.float()
        # k and v of a chunk travel as one message
        pieces = [torch.stack((kc, vc)) for kc, vc in zip(k.chunk(path_num, 0), v.chunk(path_num, 0))]
        for _ in range(1, n):
            pieces = _exchange(pieces, strides, ranks, me, group)
            kb = torch.cat([p[0] for p in pieces], 0)
            vb = torch.cat([p[1] for p in pieces], 0)
            o, l, _ = A.attn_fwd_block(q, kb, vb, False, softmax_scale)
            out, lse = A.merge_lse(out, lse, o, l.float())
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.group, ctx.ranks, ctx.path_num, ctx.scale = group, ranks, path_num, softmax_scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, ranks, P, scale = ctx.group, ctx.ranks, ctx.path_num, ctx.scale
        n = len(ranks)
        me = ranks.index(dist.get_rank())
        strides = hamilton_strides(n, P)
        dout = dout.contiguous()
        fwd_ctx = "sm100" if (q.is_cuda and A.get_backend(q) == "sm100") else None

        def block_bwd(kb, vb):
            if fwd_ctx is None and q.is_cuda and A.get_backend(q) != "ref":
                return A.attn_bwd_ref(dout, q, kb, vb, out, lse, False, scale)
            return A.attn_bwd_block(dout, q, kb, vb, out, lse, False, scale, ctx=fwd_ctx)

        dq, dk0, dv0 = block_bwd(k, v)
        dq = dq.float()
        # [k, v, dk, dv] of a chunk travel together; the gradients accumulate in fp32
        pieces = [torch.stack((kc.float(), vc.float(), dkc.float(), dvc.float()))
                  for kc, vc, dkc, dvc in zip(k.chunk(P, 0), v.chunk(P, 0), dk0.chunk(P, 0), dv0.chunk(P, 0))]
        L = k.shape[0] // P
        for _ in range(1, n):
            pieces = _exchange(pieces, strides, ranks, me, group)
            kb = torch.cat([p[0] for p in pieces], 0).to(k.dtype)
            vb = torch.cat([p[1] for p in pieces], 0).to(v.dtype)
            dq_t, dk_t, dv_t = block_bwd(kb, vb)
            dq += dq_t.float()
            for p in range(P):
                pieces[p][2] += dk_t[p * L:(p + 1) * L].float()
                pieces[p][3] += dv_t[p * L:(p + 1) * L].float()
        # after n-1 hops a chunk sits one hop before its origin on its cycle: one more hop brings the gradients home
        grads = _exchange([p[2:4].contiguous() for p in pieces], strides, ranks, me, group)
        dk = torch.cat([g[0] for g in grads], 0).to(k.dtype)
        dv = torch.cat([g[1] for g in grads], 0).to(v.dtype)
        return dq.to(q.dtype), dk, dv, None, None, None, None


def hamilton_attention(q, k, v, config=None, causal=False, softmax_scale=None, group=None, ranks=None, path_num=None):
    """q [s_local, b, nq, d], k / v [s_local, b, nkv, d]; every rank holds one contiguous 1/cp slice of the sequence."""
    if causal:
        raise NotImplementedError("Hamilton attention supports full (non-causal) attention only")
    if group is None:
        group = ps.get_context_parallel_group()
        ranks = ps.get_context_parallel_global_ranks()
    n = len(ranks)
    if path_num is None:
        path_num = int(getattr(config, "hamilton_path_num", 0) or 0) if config is not None else 0
    if path_num <= 0:
        path_num = max_paths(n)
        while path_num > 1 and k.shape[0] % path_num != 0:
            path_num -= 1
    if n == 1:
        return A.attn_fwd_block(q, k, v, False, softmax_scale)[0] if not q.requires_grad else \
            A.flash_attention(q, k, v, causal=False, softmax_scale=softmax_scale)
    return _HamiltonAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, list(ranks), path_num, softmax_scale)
