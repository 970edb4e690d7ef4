"""Ulysses context parallelism for arbitrary attention modules of the engine.

Models written against ``torch.nn.functional.scaled_dot_product_attention`` need no change: inside
``ulysses_attention_patch(group)`` that function receives ``q, k, v [b, n, s / p, d]`` (every rank holds a slice of the
sequence), exchanges sequence for heads with one all-to-all per operand (``[b, n / p, s, d]``), runs the ordinary attention on
the full sequence with its share of the heads and exchanges back.  K / V with fewer heads than the group (grouped-query
attention) are repeated up to the group size first.  ``shard_sequence`` / ``gather_sequence`` cut and restore the sequence axis
of the model's inputs and outputs; the causal mask is the attention call's own ``is_causal`` (explicit masks would have to be
full-sequence and are refused).
reference: ``context_parallel_size`` / ``ulysses_parallel_size`` of mindspeed/fsdp/parallel_engine_config.py:70-76 and the
engine's attention patch; the all-to-all layout of mindspeed/core/context_parallel/ulysses_context_parallel/
ulysses_context_parallel.py:83-108.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import mappings as M


def shard_sequence(x: torch.Tensor, group, dim: int = 1) -> torch.Tensor:
    p, r = dist.get_world_size(group), dist.get_rank(group)
    if x.shape[dim] % p != 0:
        raise ValueError(f"sequence length {x.shape[dim]} is not divisible by the context-parallel size {p}")
    return x.chunk(p, dim=dim)[r].contiguous()


def gather_sequence(x: torch.Tensor, group, dim: int = 1) -> torch.Tensor:
    """All-gather along the sequence axis (gradient: the local slice of the incoming gradient)."""
    xt = x.movedim(dim, 0).contiguous()
    out = M.gather_from_sequence_parallel_region(xt, False, group)
    return out.movedim(0, dim)


def _seq_to_heads(x, group):
    """[b, n, s/p, d] -> [b, n/p, s, d]"""
    p = dist.get_world_size(group)
    b, n, sl, d = x.shape
    t = x.reshape(b, p, n // p, sl, d).permute(1, 3, 0, 2, 4).contiguous().reshape(p * sl, b, n // p, d)
    t = M.all_to_all(group, t)                                   # rows ordered by source rank = sequence slice
    return t.permute(1, 2, 0, 3)


def _heads_to_seq(x, group):
    """[b, n/p, s, d] -> [b, n, s/p, d]"""
    p = dist.get_world_size(group)
    b, nl, s, d = x.shape
    t = M.all_to_all(group, x.permute(2, 0, 1, 3).contiguous())   # [p * s/p, b, n/p, d] by source = head group
    return t.reshape(p, s // p, b, nl, d).permute(2, 0, 3, 1, 4).reshape(b, p * nl, s // p, d)


@contextlib.contextmanager
def ulysses_attention_patch(group):
    p = dist.get_world_size(group) if group is not None else 1
    if p == 1:
        yield
        return
    orig = F.scaled_dot_product_attention

    def sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, **kw):
        if query.dim() != 4:
            return orig(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale, **kw)
        if attn_mask is not None:
            raise NotImplementedError("Ulysses context parallelism takes is_causal, not an explicit mask")
        n, nkv = query.shape[1], key.shape[1]
        if n % p != 0:
            raise ValueError(f"{n} attention heads are not divisible by the context-parallel size {p}")
        if nkv % p != 0:
            if p % nkv != 0 and nkv % p != 0:
                raise ValueError(f"{nkv} key / value heads and context-parallel size {p}: one must divide the other")
            rep = p // nkv
            key, value = key.repeat_interleave(rep, dim=1), value.repeat_interleave(rep, dim=1)
        q, k, v = (_seq_to_heads(t, group) for t in (query, key, value))
        kw.pop("enable_gqa", None)
        if k.shape[1] != q.shape[1]:
            g = q.shape[1] // k.shape[1]
            k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
        o = orig(q, k, v, dropout_p=dropout_p, is_causal=is_causal, scale=scale)
        return _heads_to_seq(o, group)
    F.scaled_dot_product_attention = sdpa
    try:
        yield
    finally:
        F.scaled_dot_product_attention = orig
