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


# ---- sequence lengths that the group size does not divide -------------------------------------------------------------
class GatherSizeCalculator:
    """Tells ``ulysses_attention`` the length of the full sequence when the ranks hold slices of different lengths;
    ``calculate()`` returns that length or None (None = every rank holds the same number of tokens)."""

    def calculate(self, *args, **kwargs):
        raise NotImplementedError


class DefaultGatherSizeCalculator(GatherSizeCalculator):
    def calculate(self, *args, **kwargs):
        return None


class DynamicGatherSizeCalculator(GatherSizeCalculator):
    """Length of the current batch's sequence, read from its attention mask (last axis) or given directly."""

    def calculate(self, *args, **kwargs):
        mask = kwargs.get("attention_mask", args[0] if args else None)
        if mask is None:
            return None
        return int(mask) if isinstance(mask, int) else int(mask.shape[-1])


def split_lengths(total: int, p: int):
    """How ``total`` tokens are laid out over ``p`` ranks when ``p`` does not divide it: the first ``total % p`` ranks hold
    one token more."""
    base, extra = divmod(total, p)
    return [base + (1 if r < extra else 0) for r in range(p)]


def seq_to_heads_unaligned(x, group, lengths):
    """[s_r, b, n, d] with s_r = lengths[rank] -> [sum(lengths), b, n/p, d]: the all-to-all receives ``lengths[j]`` rows from
    rank j (reference: the gather-size path of ulysses_context_parallel.py:127-221)."""
    p = dist.get_world_size(group)
    sl, b, n, d = x.shape
    r = dist.get_rank(group)
    if sl != lengths[r]:
        raise ValueError(f"rank {r} holds {sl} tokens, the layout says {lengths[r]}")
    t = x.reshape(sl, b, p, n // p, d).permute(2, 0, 1, 3, 4).contiguous().reshape(p * sl, b, n // p, d)
    return M.all_to_all(group, t, list(lengths), [sl] * p)


def heads_to_seq_unaligned(x, group, lengths):
    """[sum(lengths), b, n/p, d] -> [lengths[rank], b, n, d]"""
    p = dist.get_world_size(group)
    s, b, nl, d = x.shape
    r = dist.get_rank(group)
    mine = lengths[r]
    t = M.all_to_all(group, x.contiguous(), [mine] * p, list(lengths))          # [p * mine, b, n/p, d] by head group
    return t.reshape(p, mine, b, nl, d).permute(1, 2, 0, 3, 4).reshape(mine, b, p * nl, d)


def ulysses_attention(q, k, v, config, group, causal=True, softmax_scale=None, layer_number=1, inner=None,
                      gather_size_calculator: GatherSizeCalculator = None, **calc_kwargs):
    p = dist.get_world_size(group)
    nkv = k.shape[2]
    total = gather_size_calculator.calculate(**calc_kwargs) if gather_size_calculator is not None else None
    if total is not None and p > 1 and (total % p != 0 or q.shape[0] * p != total):
        # ranks hold slices of different lengths: all-to-alls with per-rank row counts
        lengths = split_lengths(total, p)
        if nkv < p:
            rep = p // nkv
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        qh, kh, vh = (seq_to_heads_unaligned(t, group, lengths) for t in (q, k, v))
        if inner is not None:
            o = inner(qh, kh, vh)
        else:
            want = getattr(config, "attention_backend", "auto") if config is not None else "library"
            backend = "library" if want == "library" else (
                "sm100" if (config is not None and config.optimization_level >= 1 and q.is_cuda) else None)
            o = A.flash_attention(qh, kh, vh, causal=causal, softmax_scale=softmax_scale, backend=backend)
        return heads_to_seq_unaligned(o, group, lengths)
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
