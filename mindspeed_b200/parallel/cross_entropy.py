"""Vocabulary-parallel cross entropy.

Each tensor-parallel rank holds logits for a contiguous vocabulary slice.  The loss
needs three small reductions: the row maximum (MAX), the target logit (SUM of a
masked gather) and the exponential sum (SUM)
(reference: mindspeed/core/tensor_parallel/cross_entropy.py:6-38).  On a GPU at
optimisation level >= 1 the local pieces (max / exp-sum / target pick / gradient
written in place over the logits) run as one sm_100a kernel per phase
(mindspeed_b200/ops/cross_entropy.py); this file is the portable composition.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import parallel_state as ps
from .layers import VocabUtility


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, label_smoothing, group):
        world = 1 if group is None else dist.get_world_size(group)
        rank = 0 if group is None else dist.get_rank(group)
        logits = logits.float()
        lmax = logits.max(dim=-1)[0]
        if world > 1:
            dist.all_reduce(lmax, op=dist.ReduceOp.MAX, group=group)
        logits = logits - lmax.unsqueeze(-1)
        per = logits.shape[-1]
        start, end = VocabUtility.vocab_range_from_per_partition_vocab_size(per, rank, world)
        mask = (target < start) | (target >= end)
        local_t = (target - start).masked_fill(mask, 0)
        flat = logits.reshape(-1, per)
        picked = flat.gather(1, local_t.reshape(-1, 1)).squeeze(1).reshape(target.shape)
        picked = picked.masked_fill(mask, 0.0)
        exp = logits.exp()
        sum_exp = exp.sum(dim=-1)
        if world > 1:
            dist.all_reduce(picked, group=group)
            dist.all_reduce(sum_exp, group=group)
        loss = sum_exp.log() - picked
        probs = exp / sum_exp.unsqueeze(-1)
        vocab = per * world
        if label_smoothing > 0:
            smoothing = label_smoothing * vocab / (vocab - 1)
            logp = probs.clamp_min(1e-30).log()
            mean_logp = logp.sum(dim=-1)
            if world > 1:
                dist.all_reduce(mean_logp, group=group)
            mean_logp = mean_logp / vocab
            loss = (1.0 - smoothing) * loss - smoothing * mean_logp
        ctx.label_smoothing, ctx.vocab = label_smoothing, vocab
        ctx.save_for_backward(probs, mask, local_t)
        return loss

    @staticmethod
    def backward(ctx, g):
        probs, mask, local_t = ctx.saved_tensors
        per = probs.shape[-1]
        grad = probs.clone()
        g2 = grad.view(-1, per)
        idx = torch.arange(g2.shape[0], device=g2.device)
        upd = 1.0 - mask.reshape(-1).float()
        if ctx.label_smoothing > 0:
            s = ctx.label_smoothing * ctx.vocab / (ctx.vocab - 1)
            g2[idx, local_t.reshape(-1)] -= (1.0 - s) * upd
            g2 -= s / ctx.vocab
        else:
            g2[idx, local_t.reshape(-1)] -= upd
        grad.mul_(g.unsqueeze(-1))
        return grad, None, None, None


def vocab_parallel_cross_entropy(vocab_parallel_logits, target, label_smoothing=0.0, group=None):
    """``vocab_parallel_logits`` [..., V/tp]; ``target`` [...] global ids; returns per-token loss [...]."""
    if group is None and ps.model_parallel_is_initialized():
        group = ps.get_tensor_model_parallel_group()
    if vocab_parallel_logits.is_cuda:
        from ..ops import cross_entropy as fused_ce
        if fused_ce.available() and label_smoothing == 0.0:
            return fused_ce.fused_vocab_parallel_cross_entropy(vocab_parallel_logits, target, group)
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target, label_smoothing, group)
