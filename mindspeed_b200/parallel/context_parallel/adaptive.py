"""Adaptive context parallelism for arbitrary attention masks.

The global mask is coarsened to rank granularity (is any key of rank j visible to any query of rank i?), the needed
KV exchanges are scheduled greedily into rounds with at most ``comm_limit`` sends and receives per rank, and each
rank merges the partial attention results of its local block and of every received block by log-sum-exp.  A k-means
pass over the coarse mask can re-order sequence blocks across ranks beforehand so that fewer exchanges are needed.
Host algorithms are native (csrc/host/adaptive_cp.cpp).
reference: mindspeed/core/context_parallel/adaptive_context_parallel/adaptive_context_parallel.py:50-371,
mindspeed/core/context_parallel/utils.py:362-708.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ...ops import attention as A
from ...utils.host_lib import host_lib
from .. import parallel_state as ps

_GLOBAL_MASK = {"mask": None, "blocks": None}
_SCHEDULE_CACHE = {}


def set_global_attention_mask(mask: torch.Tensor):
    """[S, S] bool, True = masked out."""
    _GLOBAL_MASK["mask"] = mask


def set_block_mask_list(blocks):
    """``--adaptive-cp-manually-set-mask-list``: the mask given block by block instead of as one [S, S] tensor.
    ``blocks[i][j]`` is the [s_local, s_local] bool mask (True = masked out) between the queries of context-parallel rank i
    and the keys of rank j, or None when no query of rank i sees any key of rank j; the exchange schedule is derived from
    which entries exist, so a long sequence never needs its full mask in one piece
    (reference: mindspeed/core/context_parallel/utils.py, the manually set mask list of adaptive CP)."""
    _GLOBAL_MASK["blocks"] = blocks


def coarsen_mask(visible: torch.Tensor, block: int, threads: int = 4) -> torch.Tensor:
    """visible [S, S] bool/uint8 (1 = may attend) -> [S/block, S/block] uint8."""
    v = np.ascontiguousarray(visible.to(torch.uint8).cpu().numpy())
    S = v.shape[0]
    nb = S // block
    out = np.zeros((nb, nb), dtype=np.uint8)
    host_lib().msb_coarsen_mask(v.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(S), ctypes.c_int64(block),
                                out.ctypes.data_as(ctypes.c_void_p), threads)
    return torch.from_numpy(out)


def search_kmeans(coarse: torch.Tensor, k: int, iters: int = 8, seed: int = 0) -> List[int]:
    c = np.ascontiguousarray(coarse.to(torch.uint8).cpu().numpy())
    nb = c.shape[0]
    order = np.zeros(nb, dtype=np.int64)
    host_lib().msb_search_kmeans(c.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(nb), k, iters, ctypes.c_uint64(seed),
                                 order.ctypes.data_as(ctypes.c_void_p))
    return order.tolist()


def schedule_rounds(need: torch.Tensor, comm_limit: int = 1) -> Tuple[int, torch.Tensor]:
    n = np.ascontiguousarray(need.to(torch.uint8).cpu().numpy())
    cp = n.shape[0]
    out = np.full((cp, cp), -1, dtype=np.int32)
    rounds = host_lib().msb_schedule_rounds(n.ctypes.data_as(ctypes.c_void_p), cp, comm_limit, out.ctypes.data_as(ctypes.c_void_p))
    return rounds, torch.from_numpy(out)


class _Exchange(torch.autograd.Function):
    """One round of KV block exchange: send my block to ``dsts`` and receive the blocks of ``srcs``; backward returns
    the gradients of the received blocks to their owners."""

    @staticmethod
    def forward(ctx, kv, srcs, dsts, group, ranks):
        ctx.meta = (srcs, dsts, group, ranks, kv.shape, kv.dtype)
        ctx.dev = kv.device
        bufs = [torch.empty_like(kv) for _ in srcs]
        ops = [dist.P2POp(dist.isend, kv.contiguous(), ranks[d], group) for d in dsts]
        ops += [dist.P2POp(dist.irecv, b, ranks[s], group) for s, b in zip(srcs, bufs)]
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        # the trailing token keeps this node in every rank's graph, so backward (which is collective) always runs
        return tuple(bufs) + (kv.new_zeros(1),)

    @staticmethod
    def backward(ctx, *grads):
        srcs, dsts, group, ranks, shape, dtype = ctx.meta
        grads = [g if g is not None else torch.zeros(shape, dtype=dtype, device=ctx.dev) for g in grads[:-1]]
        back = [torch.empty(shape, dtype=dtype, device=ctx.dev) for _ in dsts]
        ops = [dist.P2POp(dist.isend, g.contiguous(), ranks[s], group) for s, g in zip(srcs, grads)]
        ops += [dist.P2POp(dist.irecv, b, ranks[d], group) for d, b in zip(dsts, back)]
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        total = None
        for b in back:
            total = b if total is None else total + b
        if total is None:
            total = torch.zeros(shape, dtype=dtype, device=ctx.dev)
        return total, None, None, None, None


def adaptive_attention(q, k, v, config=None, attention_mask=None, softmax_scale=None, comm_limit: Optional[int] = None):
    """q/k/v [s_local, b, n, d] holding the contiguous sequence chunk of this context-parallel rank; the global mask
    [S, S] (True = masked) comes from ``attention_mask`` or ``set_global_attention_mask``."""
    group = ps.get_context_parallel_group()
    ranks = ps.get_context_parallel_global_ranks()
    cp, r = len(ranks), ps.get_context_parallel_rank()
    s_local = q.shape[0]
    dev = q.device
    limit = comm_limit or int(getattr(config, "adaptive_cp_comm_limit", 1) or 1)
    dynamic = bool(getattr(config, "adaptive_cp_dynamic_attn_mask", False))
    blocks = _GLOBAL_MASK["blocks"] if bool(getattr(config, "adaptive_cp_manually_set_mask_list", False)) or \
        (attention_mask is None and _GLOBAL_MASK["mask"] is None) else None
    if blocks is not None:
        need = torch.tensor([[0 if blocks[i][j] is None else 1 for j in range(cp)] for i in range(cp)], dtype=torch.uint8)
        key = ("blocks", id(blocks), limit)

        def sub_mask(qr, kr):
            return blocks[qr][kr].to(dev).view(1, 1, s_local, s_local)
    else:
        mask = attention_mask if attention_mask is not None and attention_mask.dim() == 2 else _GLOBAL_MASK["mask"]
        if mask is None:
            raise RuntimeError("adaptive context parallelism needs the global [S, S] attention mask or a block mask list")
        key = ("mask", mask.data_ptr(), mask._version, tuple(mask.shape), s_local, limit)
        if not dynamic and key in _SCHEDULE_CACHE:
            need = _SCHEDULE_CACHE[key][2]
        else:
            need = coarsen_mask(~mask.bool(), s_local)              # [cp, cp]

        def sub_mask(qr, kr):
            return mask[qr * s_local:(qr + 1) * s_local, kr * s_local:(kr + 1) * s_local].to(dev).view(1, 1, s_local, s_local)
    if not dynamic and key in _SCHEDULE_CACHE:
        n_rounds, round_of, _ = _SCHEDULE_CACHE[key]
    else:
        n_rounds, round_of = schedule_rounds(need, limit)
        if not dynamic:
            if len(_SCHEDULE_CACHE) > 16:
                _SCHEDULE_CACHE.clear()
            _SCHEDULE_CACHE[key] = (n_rounds, round_of, need)

    out = lse = None
    if need[r, r]:
        out, lse = A.attention_ref(q, k, v, causal=False, softmax_scale=softmax_scale, mask=sub_mask(r, r), return_lse=True)
    kv = torch.stack((k, v))
    tokens = []
    for rd in range(n_rounds):
        srcs = [j for j in range(cp) if round_of[r, j] == rd]          # blocks I receive this round
        dsts = [i for i in range(cp) if round_of[i, r] == rd]          # ranks that need my block this round
        got = _Exchange.apply(kv, srcs, dsts, group, ranks)
        tokens.append(got[-1])
        for j, blk in zip(srcs, got[:-1]):
            o, l = A.attention_ref(q, blk[0], blk[1], causal=False, softmax_scale=softmax_scale, mask=sub_mask(r, j), return_lse=True)
            if out is None:
                out, lse = o, l
            else:
                out, lse = A.merge_lse(out, lse, o, l)
    if out is None:
        out = torch.zeros(q.shape[0], q.shape[1], q.shape[2], v.shape[-1], dtype=q.dtype, device=dev) + q.sum() * 0
    for t in tokens:
        out = out + (t.sum() * 0).to(out.dtype)
    return out
