"""Slicing a batch along the sequence for context parallelism.

ring (``megatron_cp_algo``): causal load balancing — the sequence is cut in 2*cp chunks and rank r
  keeps chunks r and 2*cp-1-r, so every ring step does the same amount of work;
ulysses / kv-allgather: contiguous chunk r;
hybrid: ring split over the ring degree first, then a contiguous Ulysses chunk inside.
(reference: mindspeed/core/context_parallel/get_batch_utils.py:89-137,244-277,310-334)
"""
from __future__ import annotations

import torch

from .. import parallel_state as ps

_SEQ_DIM = {"tokens": 1, "labels": 1, "loss_mask": 1, "position_ids": 1, "attention_mask": 2}


def _ring_slice(val, seq_dim, cp, r):
    shp = list(val.shape)
    v = val.view(*shp[:seq_dim], 2 * cp, shp[seq_dim] // (2 * cp), *shp[seq_dim + 1:])
    idx = torch.tensor([r, 2 * cp - 1 - r], device=val.device)
    v = v.index_select(seq_dim, idx)
    return v.reshape(*shp[:seq_dim], -1, *shp[seq_dim + 1:])


def _contig_slice(val, seq_dim, cp, r):
    return val.chunk(cp, dim=seq_dim)[r].contiguous()


def slice_for_cp(val, seq_dim, algo, cp=None, r=None):
    cp = ps.get_context_parallel_world_size() if cp is None else cp
    r = ps.get_context_parallel_rank() if r is None else r
    if cp == 1 or val is None:
        return val
    if algo in ("ulysses_cp_algo",):
        return _contig_slice(val, seq_dim, cp, r)
    if algo in ("hybrid_cp_algo", "hybrid_adaptive_cp_algo"):
        u = ps.get_context_parallel_for_hybrid_ulysses_world_size()
        ur = ps.get_context_parallel_for_hybrid_ulysses_rank()
        ring, rr = ps.get_context_parallel_for_hybrid_ring_world_size(), ps.get_context_parallel_for_hybrid_ring_rank()
        v = _ring_slice(val, seq_dim, ring, rr)
        return _contig_slice(v, seq_dim, u, ur)
    if algo in ("adaptive_cp_algo", "hamilton_cp_algo"):       # full attention: no causal balancing, contiguous slices
        return _contig_slice(val, seq_dim, cp, r)
    return _ring_slice(val, seq_dim, cp, r)  # megatron_cp_algo, kvallgather (2-chunk, causal balanced)


def hybrid_local_positions(full_len, device):
    pos = torch.arange(full_len, device=device).view(1, -1)
    return slice_for_cp(pos, 1, "hybrid_cp_algo").view(-1)


def get_batch_on_this_cp_rank(batch, algo=None):
    cp = ps.get_context_parallel_world_size() if ps.model_parallel_is_initialized() else 1
    if cp == 1:
        return batch
    if algo is None:
        try:
            from ...training.global_vars import get_args
            algo = get_args().context_parallel_algo
        except Exception:
            algo = "megatron_cp_algo"
    out = {}
    for k, v in batch.items():
        out[k] = slice_for_cp(v, _SEQ_DIM.get(k, 1), algo) if v is not None else None
    return out
