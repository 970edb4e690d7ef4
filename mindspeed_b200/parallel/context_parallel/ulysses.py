"""Ulysses context parallelism: all-to-all sequence <-> heads around ordinary attention.

q/k/v arrive [s/p, b, n, d]; an all-to-all makes them [s, b, n/p, d]; attention runs on the full sequence with a
head subset; a second all-to-all restores [s/p, b, n*d]
(reference: mindspeed/core/context_parallel/ulysses_context_parallel/ulysses_context_parallel.py:83-108,127-221).
GQA with fewer KV heads than ranks repeats KV heads up to the group size first (:186-190).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...ops import attention as A
from .. import mappings as M


_FUSED = {"on": False}


def set_fused_all_to_all(flag: bool):
    """Optimisation level 2: the exchanges run as peer-memory pull kernels with the layout transform folded in
    (mindspeed_b200/ops/ulysses_comm.py) instead of permute + NCCL all-to-all."""
    _FUSED["on"] = bool(flag)


def _use_fused(x, group):
    if not _FUSED["on"]:
        return False
    from ...ops import ulysses_comm as U
    return U.eligible(x, group) and (x.shape[-1] * x.element_size() * (x.shape[2] if x.dim() == 4 else 1)) % 16 == 0


def seq_to_heads(x, group):
    """[s/p, b, n, d] -> [s, b, n/p, d]"""
    p = dist.get_world_size(group)
    if p == 1:
        return x
    if _use_fused(x, group) and (x.shape[2] // p) * x.shape[3] * x.element_size() % 16 == 0:
        from ...ops.ulysses_comm import seq_to_heads_fused
        return seq_to_heads_fused(x, group)
    sl, b, n, d = x.shape
    t = x.reshape(sl, b, p, n // p, d).permute(2, 0, 1, 3, 4).contiguous()  # [p, s/p, b, n/p, d]
    t = M.all_to_all(group, t.reshape(p * sl, b, n // p, d))
    return t  # rows are now ordered by source rank = sequence chunk


def heads_to_seq(x, group):
    """[s, b, n/p, d] -> [s/p, b, n, d]"""
    p = dist.get_world_size(group)
    if p == 1:
        return x
    if _use_fused(x, group):
        from ...ops.ulysses_comm import heads_to_seq_fused
        return heads_to_seq_fused(x, group)
    s, b, nl, d = x.shape
    t = M.all_to_all(group, x.contiguous())                                   # [p * s/p, b, n/p, d] by source = head group
    t = t.reshape(p, s // p, b, nl, d).permute(1, 2, 0, 3, 4).contiguous()    # [s/p, b, p, n/p, d]
    return t.reshape(s // p, b, p * nl, d)


def ulysses_attention(q, k, v, config, group, causal=True, softmax_scale=None, layer_number=1, inner=None):
    p = dist.get_world_size(group)
    nkv = k.shape[2]
    if nkv < p and bool(getattr(config, "use_ulysses_allgather_kv", False)) and p % nkv == 0:
        # --use-ulysses-allgather-kv: fewer KV heads than ranks.  Instead of repeating the KV heads up to the group size
        # and sending the copies through the all-to-all, gather K and V along the sequence (gradient: reduce-scatter) and
        # keep only the KV head this rank's query heads use (reference: ulysses_context_parallel.py:456-557,589-595)
        qh = seq_to_heads(q, group)
        r = dist.get_rank(group)
        kv_idx = r * nkv // p
        # gather every KV head (each rank must contribute the same heads), then keep the one this rank's queries use;
        # the other heads get zero gradient here and their real gradient from the ranks that use them
        kh = M.gather_from_sequence_parallel_region(k.contiguous(), True, group)[:, :, kv_idx:kv_idx + 1]
        vh = M.gather_from_sequence_parallel_region(v.contiguous(), True, group)[:, :, kv_idx:kv_idx + 1]
    else:
        if nkv < p:
            rep = p // nkv
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        qh, kh, vh = seq_to_heads(q, group), seq_to_heads(k, group), seq_to_heads(v, group)
    if inner is not None:
        o = inner(qh, kh, vh)
    else:
        want = getattr(config, "attention_backend", "auto") if config is not None else "library"
        backend = "library" if want == "library" else (
            "sm100" if (config is not None and config.optimization_level >= 1 and q.is_cuda) else None)
        o = A.flash_attention(qh, kh, vh, causal=causal, softmax_scale=softmax_scale, backend=backend)
    return heads_to_seq(o, group)
