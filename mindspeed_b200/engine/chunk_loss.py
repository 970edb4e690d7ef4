"""Chunked language-model loss: cross entropy of ``hidden @ weight^T`` without ever holding the [tokens, vocab] logits.

The forward walks over chunks of tokens; for each chunk it forms the logits, the loss contribution and - immediately -
the gradients with respect to the hidden states and the output weight, then drops the logits.  Peak extra memory is
one chunk of logits instead of all of them (for vocab 128k and 8k tokens: 64 MB per 256-token chunk instead of 4 GB in
fp32).  The backward only scales the stored gradients by the incoming loss gradient.
reference: mindspeed/fsdp/memory/chunk_loss/chunk_loss.py:6-252.
"""
from __future__ import annotations

from typing import Optional

import torch


class _ChunkedLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, chunk, ignore_index, reduction):
        T = hidden.shape[0]
        need_h, need_w = hidden.requires_grad, weight.requires_grad
        gh = torch.zeros_like(hidden) if need_h else None
        gw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if need_w else None
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        valid = (labels != ignore_index)
        n_valid = valid.sum().clamp(min=1).float()
        denom = n_valid if reduction == "mean" else torch.ones((), device=hidden.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            h = hidden[s:e]
            logits = (h @ weight.t()).float()
            lab = labels[s:e]
            m = valid[s:e]
            lse = torch.logsumexp(logits, dim=-1)
            tgt = logits.gather(1, lab.clamp(min=0).unsqueeze(1)).squeeze(1)
            total += ((lse - tgt) * m).sum()
            if need_h or need_w:
                p = torch.softmax(logits, dim=-1)
                p.scatter_add_(1, lab.clamp(min=0).unsqueeze(1), -torch.ones_like(tgt).unsqueeze(1))
                p.mul_((m.float() / denom).unsqueeze(1))
                pd = p.to(hidden.dtype)
                if need_h:
                    gh[s:e] = pd @ weight
                if need_w:
                    gw.addmm_(pd.t().float(), h.float())
            del logits
        ctx.save_for_backward(gh, gw)
        ctx.w_dtype = weight.dtype
        return total / denom

    @staticmethod
    def backward(ctx, g):
        gh, gw = ctx.saved_tensors
        return (gh * g.to(gh.dtype) if gh is not None else None, (gw * g).to(ctx.w_dtype) if gw is not None else None,
                None, None, None, None)


def chunked_lm_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, chunk_size: Optional[int] = 1024,
                    ignore_index: int = -100, reduction: str = "mean") -> torch.Tensor:
    """hidden [..., H], weight [V, H], labels [...] -> scalar loss ("mean" over non-ignored tokens or "sum")."""
    if reduction not in ("mean", "sum"):
        raise ValueError("reduction must be 'mean' or 'sum'")
    h = hidden.reshape(-1, hidden.shape[-1])
    lab = labels.reshape(-1)
    chunk = h.shape[0] if not chunk_size else int(chunk_size)
    return _ChunkedLoss.apply(h, weight, lab, max(1, chunk), ignore_index, reduction)
