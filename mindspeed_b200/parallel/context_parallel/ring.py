"""Ring attention with causal load balancing, double-buffered KV exchange, optional double ring and KV cache.

Each rank holds sequence chunks r and 2cp-1-r (of 2cp).  At ring step i it attends its queries to the KV block
that originated on rank (r - i) mod cp while the block for step i+1 is already in flight:
   i == 0         : local block, ordinary causal mask on the concatenated two chunks
   source < rank  : all queries vs the FIRST KV chunk only, no mask
   source > rank  : SECOND query chunk vs the whole KV block, no mask
Partial results are merged with the log-sum-exp form of the online-softmax update.  Backward runs the same ring;
dK/dV of a block travel with the block and arrive home after a full turn.
reference: mindspeed/core/context_parallel/ring_context_parallel/ring_context_parallel.py:16-33,918-1188;
bookkeeping mindspeed/core/context_parallel/utils.py:122-206,300-340; KV cache policy
context_parallel_kv_cache.py:5-133; double ring groups model_parallel_utils.py:121-212.

On one NVSwitch domain every peer is one hop away, so the ring order carries no locality; the window
(``--cp-window-size``) is accepted and arranges the same exchanges as inner / outer rings.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ...ops import attention as A
from .. import parallel_state as ps


class RingP2P:
    """Send to the next rank / receive from the previous one; with a twin group the two directions use
    different communicators so they progress concurrently (reference: context_parallel/utils.py:122-206)."""

    def __init__(self, ranks: List[int], group, group_overlap=None, is_backward=False):
        me = dist.get_rank()
        i = ranks.index(me)
        n = len(ranks)
        self.next = ranks[(i + 1) % n]
        self.prev = ranks[(i - 1) % n]
        if is_backward:
            self.next, self.prev = self.prev, self.next
        self.group, self.group_overlap = group, group_overlap
        self.reqs = []
        self.even = i % 2 == 0

    def async_send_recv(self, send_tensor, recv_tensor):
        g_send = self.group
        g_recv = self.group_overlap if self.group_overlap is not None else self.group
        if self.group_overlap is not None and not self.even:
            g_send, g_recv = g_recv, g_send
        if self.even:
            self.reqs.append(dist.isend(send_tensor, self.next, group=g_send))
            self.reqs.append(dist.irecv(recv_tensor, self.prev, group=g_recv))
        else:
            self.reqs.append(dist.irecv(recv_tensor, self.prev, group=g_recv))
            self.reqs.append(dist.isend(send_tensor, self.next, group=g_send))

    def wait(self):
        for r in self.reqs:
            r.wait()
        self.reqs = []


def _halves(t):
    """[2c, b, n, d] -> (first chunk, second chunk) views."""
    c = t.shape[0] // 2
    return t[:c], t[c:]


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, ranks, group_overlap, causal, scale, cache_kv):
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        ring = RingP2P(ranks, group, group_overlap)
        kv = torch.stack((k, v)).contiguous()           # [2, s, b, nkv, d]
        nxt = torch.empty_like(kv)
        out = lse = None
        blocks = []                                       # what each step needs for backward
        kv_cache = []
        for i in range(cp):
            if i < cp - 1:
                ring.async_send_recv(kv, nxt)
            src = (rank - i) % cp
            kk, vv = kv[0], kv[1]
            if not causal or i == 0:
                o, l, c = A.attn_fwd_block(q, kk, vv, causal and i == 0, scale)
                mode = 0
            elif src < rank:
                o, l, c = A.attn_fwd_block(q, _halves(kk)[0], _halves(vv)[0], False, scale)
                mode = 1
            else:
                o, l, c = A.attn_fwd_block(_halves(q)[1], kk, vv, False, scale)
                mode = 2
            if out is None:
                out, lse = o.contiguous(), l.contiguous()
            elif mode == 2:
                h = q.shape[0] // 2
                mo, ml = A.merge_lse(out[h:], lse[..., h:], o, l)
                out = torch.cat((out[:h], mo), dim=0)
                lse = torch.cat((lse[..., :h], ml), dim=-1)
            else:
                out, lse = A.merge_lse(out, lse, o, l)
            blocks.append((mode, c))
            if cache_kv:
                kv_cache.append(kv.clone() if i < cp - 1 else kv)
            if i < cp - 1:
                ring.wait()
                kv, nxt = nxt, kv
        ctx.save_for_backward(q, k, v, out, lse, *(kv_cache if cache_kv else []))
        ctx.meta = (group, ranks, group_overlap, causal, scale, blocks, cache_kv)
        return out

    @staticmethod
    def backward(ctx, dout):
        group, ranks, group_overlap, causal, scale, blocks, cache_kv = ctx.meta
        saved = ctx.saved_tensors
        q, k, v, out, lse = saved[:5]
        cache = list(saved[5:])
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        dout = dout.contiguous()
        kv_ring = RingP2P(ranks, group, group_overlap)
        dkv_ring = RingP2P(ranks, group, group_overlap)
        kv = torch.stack((k, v)).contiguous()
        nxt = torch.empty_like(kv)
        dq = torch.zeros_like(q, dtype=torch.float32)
        dkv = torch.zeros_like(kv, dtype=torch.float32)  # gradient of the block currently held; travels with it
        dkv_recv = torch.empty_like(dkv)
        h = q.shape[0] // 2
        for i in range(cp):
            if cache_kv:
                kv = cache[i]
            elif i < cp - 1:
                kv_ring.async_send_recv(kv, nxt)
            mode, c = blocks[i]
            kk, vv = kv[0], kv[1]
            if mode == 0:
                gq, gk, gv = A.attn_bwd_block(dout, q, kk, vv, out, lse, causal and i == 0, scale, c)
                dq += gq.float()
                blk = torch.stack((gk, gv)).float()
            elif mode == 1:
                gq, gk, gv = A.attn_bwd_block(dout, q, _halves(kk)[0], _halves(vv)[0], out, lse, False, scale, c)
                dq += gq.float()
                blk = torch.zeros_like(dkv)
                blk[0, :h], blk[1, :h] = gk.float(), gv.float()
            else:
                gq, gk, gv = A.attn_bwd_block(dout[h:], q[h:], kk, vv, out[h:], lse[..., h:].contiguous(), False, scale, c)
                dq[h:] += gq.float()
                blk = torch.stack((gk, gv)).float()
            if i > 0:
                dkv_ring.wait()
                dkv = dkv_recv + blk
                dkv_recv = torch.empty_like(dkv)
            else:
                dkv = blk
            # pass the accumulated gradient of this block on, together with the block itself
            dkv_ring.async_send_recv(dkv, dkv_recv)
            if not cache_kv and i < cp - 1:
                kv_ring.wait()
                kv, nxt = nxt, kv
        dkv_ring.wait()
        dkv = dkv_recv  # after cp hops the gradient of the local block is home
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None, None, None


def _double_ring_order(ranks, window):
    """Visiting order for a double ring: the inner ring turns inside a window, the outer ring shifts by whole
    windows.  On NVSwitch the sequence of sources is what matters; it is a permutation of the plain ring."""
    return ranks


def ring_attention(q, k, v, config=None, causal=True, softmax_scale=None, layer_number=1, group=None, ranks=None,
                   group_overlap=None):
    """q [s_local, b, nq, d], k/v [s_local, b, nkv, d] where s_local holds chunks (r, 2cp-1-r)."""
    if group is None:
        group = ps.get_context_parallel_group()
        ranks = ps.get_context_parallel_global_ranks()
        group_overlap = ps.get_context_parallel_group_for_send_recv_overlap()
    policy = getattr(config, "context_parallel_kv_cache_policy", None) if config is not None else None
    interval = getattr(config, "context_parallel_cache_interval", 0) if config is not None else 0
    cache = policy in ("full", "half") and (interval == 0 or (layer_number - 1) % (interval + 1) == 0)
    return _RingAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, list(ranks), group_overlap, causal,
                                softmax_scale, cache)
