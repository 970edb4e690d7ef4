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

``--cp-window-size w`` turns the ring into a double ring (``ring_schedule``): w - 1 hops inside a window of w ranks, then one
hop to the next window.  On one NVSwitch domain every peer is one hop away and the order carries no locality; across nodes the
window is the node, so only every w-th hop crosses the slower links.
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

    def async_send_recv(self, send_tensor, recv_tensor, dst=None, src=None):
        """Send to ``dst`` and receive from ``src`` (global ranks; default: the ring neighbours).  With explicit peers the
        two transfers go out as one batched call, which needs no even / odd ordering."""
        if dst is not None or src is not None:
            ops = [dist.P2POp(dist.isend, send_tensor, self.next if dst is None else dst, self.group),
                   dist.P2POp(dist.irecv, recv_tensor, self.prev if src is None else src, self.group)]
            self.reqs.extend(dist.batch_isend_irecv(ops))
            return
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


def _pack_kv(k, v):
    """K and V travel as one message: stacked when they have the same shape, else concatenated along the head dimension
    (multi-latent attention: K carries the rotary part, so its head dimension is larger than V's; reference:
    mindspeed/core/context_parallel/utils.py:143-197)."""
    if k.shape == v.shape:
        return torch.stack((k, v)).contiguous()
    return torch.cat((k, v), dim=-1).contiguous()


def _unpack_kv(kv, dk, same):
    if same:
        return kv[0], kv[1]
    return kv[..., :dk].contiguous(), kv[..., dk:].contiguous()


def _pack_grads(gk, gv, same):
    return torch.stack((gk, gv)).float() if same else torch.cat((gk, gv), dim=-1).float()


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, ranks, group_overlap, causal, scale, cache_kv, window=1):
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        ring = RingP2P(ranks, group, group_overlap)
        srcs, send_to, recv_from, _ = ring_schedule(cp, rank, window)
        same, dk = k.shape == v.shape, k.shape[-1]
        kv = _pack_kv(k, v)                               # [2, s, b, nkv, d], or [s, b, nkv, dk + dv]
        nxt = torch.empty_like(kv)
        out = lse = None
        blocks = []                                       # what each step needs for backward
        kv_cache = []
        for i in range(cp):
            if i < cp - 1:
                if window > 1:
                    ring.async_send_recv(kv, nxt, ranks[send_to[i]], ranks[recv_from[i]])
                else:
                    ring.async_send_recv(kv, nxt)
            src = srcs[i]
            kk, vv = _unpack_kv(kv, dk, same)
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
        ctx.meta = (group, ranks, group_overlap, causal, scale, blocks, cache_kv, window)
        return out

    @staticmethod
    def backward(ctx, dout):
        group, ranks, group_overlap, causal, scale, blocks, cache_kv, window = ctx.meta
        saved = ctx.saved_tensors
        q, k, v, out, lse = saved[:5]
        cache = list(saved[5:])
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        srcs, send_to, recv_from, home_from = ring_schedule(cp, rank, window)
        same, dk = k.shape == v.shape, k.shape[-1]
        dout = dout.contiguous()
        kv_ring = RingP2P(ranks, group, group_overlap)
        dkv_ring = RingP2P(ranks, group, group_overlap)
        kv = _pack_kv(k, v)
        nxt = torch.empty_like(kv)
        dq = torch.zeros_like(q, dtype=torch.float32)
        dkv = torch.zeros_like(kv, dtype=torch.float32)  # gradient of the block currently held; travels with it
        dkv_recv = torch.empty_like(dkv)
        h = q.shape[0] // 2
        for i in range(cp):
            if cache_kv:
                kv = cache[i]
            elif i < cp - 1:
                if window > 1:
                    kv_ring.async_send_recv(kv, nxt, ranks[send_to[i]], ranks[recv_from[i]])
                else:
                    kv_ring.async_send_recv(kv, nxt)
            mode, c = blocks[i]
            kk, vv = _unpack_kv(kv, dk, same)
            if mode == 0:
                gq, gk, gv = A.attn_bwd_block(dout, q, kk, vv, out, lse, causal and i == 0, scale, c)
                dq += gq.float()
                blk = _pack_grads(gk, gv, same)
            elif mode == 1:
                gq, gk, gv = A.attn_bwd_block(dout, q, _halves(kk)[0], _halves(vv)[0], out, lse, False, scale, c)
                dq += gq.float()
                blk = torch.zeros_like(dkv)
                if same:
                    blk[0, :h], blk[1, :h] = gk.float(), gv.float()
                else:
                    blk[:h] = torch.cat((gk, gv), dim=-1).float()
            else:
                gq, gk, gv = A.attn_bwd_block(dout[h:], q[h:], kk, vv, out[h:], lse[..., h:].contiguous(), False, scale, c)
                dq[h:] += gq.float()
                blk = _pack_grads(gk, gv, same)
            if i > 0:
                dkv_ring.wait()
                dkv = dkv_recv + blk
                dkv_recv = torch.empty_like(dkv)
            else:
                dkv = blk
            # pass the accumulated gradient of this block on, together with the block itself; after the last step it goes
            # straight to the block's origin
            if window > 1:
                if i < cp - 1:
                    dkv_ring.async_send_recv(dkv, dkv_recv, ranks[send_to[i]], ranks[recv_from[i]])
                else:
                    dkv_ring.async_send_recv(dkv, dkv_recv, ranks[srcs[i]], ranks[home_from])
            else:
                dkv_ring.async_send_recv(dkv, dkv_recv)
            if not cache_kv and i < cp - 1:
                kv_ring.wait()
                kv, nxt = nxt, kv
        dkv_ring.wait()
        dkv = dkv_recv  # the gradient of the local block is home
        if same:
            gk_home, gv_home = dkv[0], dkv[1]
        else:
            gk_home, gv_home = dkv[..., :dk], dkv[..., dk:]
        return dq.to(q.dtype), gk_home.to(k.dtype), gv_home.to(v.dtype), None, None, None, None, None, None, None


def ring_schedule(cp: int, rank: int, window: int = 1):
    """Who holds what, step by step.  Returns (src, send_to, recv_from, home_from): at step i this rank works on the block
    that originated on ``src[i]``; after the step it passes the block to ``send_to[i]`` and receives the next one from
    ``recv_from[i]`` (i < cp - 1); ``home_from`` is the rank that holds this rank's own block at the last step, i.e. where
    its dK / dV come home from.  All values are indices into the group's rank list.

    window == 1: the plain ring.  window = w > 1 (``--cp-window-size``): a double ring - w - 1 hops around the inner ring of
    the rank's window, then one hop on the outer ring to the same inner position of the next window, and so on; on
    multi-node jobs the window is chosen as the node so that only every w-th hop leaves it
    (reference: mindspeed/core/context_parallel/model_parallel_utils.py:121-212 builds the two ring groups,
    ring_context_parallel.py:918-1028 alternates them)."""
    w = max(1, int(window))
    if cp % w != 0:
        raise ValueError(f"cp_window_size {w} does not divide the context-parallel size {cp}")
    W = cp // w

    def walk(r):
        """The sequence of ranks that the block starting on r visits."""
        win, pos = divmod(r, w)
        seq = [r]
        for i in range(cp - 1):
            if w > 1 and i % w != w - 1:
                pos = (pos + 1) % w                  # inner hop
            elif w > 1:
                win = (win + 1) % W                  # outer hop
            else:
                pos, win = 0, (win + 1) % W          # plain ring over single-rank windows
            seq.append(win * w + pos)
        return seq

    walks = [walk(r) for r in range(cp)]
    src = [next(o for o in range(cp) if walks[o][i] == rank) for i in range(cp)]
    send_to = [walks[src[i]][i + 1] for i in range(cp - 1)]
    recv_from = [walks[src[i + 1]][i] for i in range(cp - 1)]
    home_from = walks[rank][cp - 1]
    return src, send_to, recv_from, home_from


class _RingAttentionUnaligned(torch.autograd.Function):
    """Ring attention without a causal mask for sequence slices of different lengths per rank (``shapes[r]`` tokens on
    rank r): every message is sized by the block that travels - the receive buffer of a step by the block that arrives,
    the gradient buffer by the block it belongs to (reference: the ``shapes`` argument of ringattn_context_parallel,
    mindspeed/core/context_parallel/ring_context_parallel/ring_context_parallel.py:422-426, 995-1028, 1104-1178)."""

    @staticmethod
    def forward(ctx, q, k, v, group, ranks, group_overlap, scale, shapes):
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        if q.shape[0] != shapes[rank] or k.shape[0] != shapes[rank]:
            raise ValueError(f"rank {rank} holds {q.shape[0]} tokens, shapes says {shapes[rank]}")
        ring = RingP2P(ranks, group, group_overlap)
        same, dk = k.shape == v.shape, k.shape[-1]
        seq_dim = 1 if same else 0
        kv = _pack_kv(k, v)

        def like(block):
            shp = list(kv.shape)
            shp[seq_dim] = shapes[block]
            return shp
        out = lse = None
        blocks = []
        for i in range(cp):
            nxt = None
            if i < cp - 1:
                nxt = kv.new_empty(like((rank - i - 1) % cp))
                ring.async_send_recv(kv, nxt)
            kk, vv = _unpack_kv(kv, dk, same)
            o, l, c = A.attn_fwd_block(q, kk, vv, False, scale)
            out, lse = (o.contiguous(), l.contiguous()) if out is None else A.merge_lse(out, lse, o, l)
            blocks.append(c)
            if i < cp - 1:
                ring.wait()
                kv = nxt
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (group, ranks, group_overlap, scale, blocks, list(shapes))
        return out

    @staticmethod
    def backward(ctx, dout):
        group, ranks, group_overlap, scale, blocks, shapes = ctx.meta
        q, k, v, out, lse = ctx.saved_tensors
        cp = len(ranks)
        rank = ranks.index(dist.get_rank())
        same, dk = k.shape == v.shape, k.shape[-1]
        seq_dim = 1 if same else 0
        dout = dout.contiguous()
        kv_ring, dkv_ring = RingP2P(ranks, group, group_overlap), RingP2P(ranks, group, group_overlap)
        kv = _pack_kv(k, v)

        def like(block, ref):
            shp = list(ref.shape)
            shp[seq_dim] = shapes[block]
            return shp
        dq = torch.zeros_like(q, dtype=torch.float32)
        dkv_recv = None
        for i in range(cp):
            nxt = None
            if i < cp - 1:
                nxt = kv.new_empty(like((rank - i - 1) % cp, kv))
                kv_ring.async_send_recv(kv, nxt)
            kk, vv = _unpack_kv(kv, dk, same)
            gq, gk, gv = A.attn_bwd_block(dout, q, kk, vv, out, lse, False, scale, blocks[i])
            dq += gq.float()
            blk = _pack_grads(gk, gv, same)
            if i > 0:
                dkv_ring.wait()
                blk = dkv_recv + blk                      # what earlier holders of this block accumulated
            # the gradient travels with its block; after the last step it arrives at the block's origin.  What arrives here
            # next belongs to the block this rank holds in the next step (its own block after the last one)
            dkv_recv = blk.new_empty(like((rank - i - 1) % cp, blk))
            dkv_ring.async_send_recv(blk, dkv_recv)
            if i < cp - 1:
                kv_ring.wait()
                kv = nxt
        dkv_ring.wait()
        if same:
            gk_home, gv_home = dkv_recv[0], dkv_recv[1]
        else:
            gk_home, gv_home = dkv_recv[..., :dk], dkv_recv[..., dk:]
        return dq.to(q.dtype), gk_home.to(k.dtype), gv_home.to(v.dtype), None, None, None, None, None


def ring_attention(q, k, v, config=None, causal=True, softmax_scale=None, layer_number=1, group=None, ranks=None,
                   group_overlap=None, shapes=None):
    """q [s_local, b, nq, d], k/v [s_local, b, nkv, d] where s_local holds chunks (r, 2cp-1-r).
    ``shapes``: tokens per rank when the slices differ in length (contiguous slices, no causal mask)."""
    if group is None:
        group = ps.get_context_parallel_group()
        ranks = ps.get_context_parallel_global_ranks()
        group_overlap = ps.get_context_parallel_group_for_send_recv_overlap()
    if shapes is not None and len(set(shapes)) > 1:
        if causal:
            raise NotImplementedError("ring attention over slices of different lengths is implemented without a causal mask")
        return _RingAttentionUnaligned.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, list(ranks), group_overlap,
                                             softmax_scale, list(shapes))
    policy = getattr(config, "context_parallel_kv_cache_policy", None) if config is not None else None
    interval = getattr(config, "context_parallel_cache_interval", 0) if config is not None else 0
    cache = policy in ("full", "half") and (interval == 0 or (layer_number - 1) % (interval + 1) == 0)
    window = int(getattr(config, "cp_window_size", 1) or 1) if config is not None else 1
    if window >= len(ranks) or len(ranks) % max(window, 1) != 0:
        window = 1
    return _RingAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, list(ranks), group_overlap, causal,
                                softmax_scale, cache, window)
