"""Attention over a per-query selection of keys (DeepSeek sparse attention): every query attends only to the top-k keys
its lightning indexer picked.

Two forms of the same function:

* ``sparse_attention`` - per-head keys and values ``k, v [B, S, H, d]``; one block of query rows builds its
  ``[B, H, tb, S]`` scores, keeps the selected columns and normalises over them.
* ``sparse_latent_attention`` - the weight-absorbed form for multi-head latent attention: the query has been taken
  through the key up-projection, so all heads read ONE latent row per key (``kv [B, S, dl]`` and the shared rotary key
  ``k_pe [B, S, dr]``); only the selected rows are gathered, ``[B, tb, K, dl + dr]`` per block, which is what makes the
  selection pay: bytes per query are K latent rows instead of S.  The caller applies the value up-projection to the
  returned latent context.

Both return the context and ``p [B, T, K]``: the attention distribution over the selected keys, averaged over heads
(the target of the indexer's KL loss).  Query rows are processed in blocks and each block is re-computed in backward
(``torch.utils.checkpoint``) so the gathers are never all resident.
reference: mindspeed/features_manager/transformer/experimental_attention_variant/dsa.py:14-22 (flags; the reference
maps them to fused sparse-flash-attention / lightning-indexer operators).
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint


def _softmax_selected(s, valid):
    """softmax over the last axis of ``s`` restricted to ``valid``; rows without any valid entry give zeros."""
    s = s.masked_fill(~valid, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True).clamp_min(1e-30)


def _blocks(fn, T, block, use_ckpt, *per_row, shared=()):
    outs = []
    for t0 in range(0, T, block):
        args = [a[:, t0:t0 + block] for a in per_row]
        if use_ckpt and torch.is_grad_enabled() and any(torch.is_tensor(a) and a.requires_grad for a in list(per_row) + list(shared)):
            outs.append(checkpoint(fn, *args, *shared, use_reentrant=False))
        else:
            outs.append(fn(*args, *shared))
    return tuple(torch.cat([o[i] for o in outs], dim=1) for i in range(len(outs[0])))


def sparse_attention(q, k, v, idx, softmax_scale: float, block: int = 512, recompute: bool = True):
    """q [B, T, H, d]; k [B, S, H, d]; v [B, S, H, dv]; idx [B, T, K] (-1 = no key) -> (out [B, T, H, dv], p [B, T, K])."""
    S = k.shape[1]

    def one(qb, ib, k, v):
        valid = ib >= 0                                                     # [B, tb, K]
        sel = torch.zeros(ib.shape[0], ib.shape[1], S + 1, dtype=torch.bool, device=ib.device)
        sel.scatter_(2, torch.where(valid, ib, torch.full_like(ib, S)), True)
        sel = sel[..., :S]
        s = torch.einsum("bthd,bshd->bhts", qb.float(), k.float()) * softmax_scale
        p = _softmax_selected(s, sel.unsqueeze(1))                          # [B, H, tb, S]
        o = torch.einsum("bhts,bshd->bthd", p, v.float()).to(qb.dtype)
        pk = torch.gather(p.mean(dim=1), 2, ib.clamp_min(0)) * valid
        return o, pk

    return _blocks(one, q.shape[1], block, recompute, q, idx, shared=(k, v))


def sparse_latent_attention(q_lat, q_pe, kv, k_pe, idx, softmax_scale: float, block: int = 256, recompute: bool = True):
    """q_lat [B, T, H, dl]; q_pe [B, T, H, dr]; kv [B, S, dl]; k_pe [B, S, dr]; idx [B, T, K]
    -> (latent context [B, T, H, dl], p [B, T, K])."""
    B = kv.shape[0]
    bi = torch.arange(B, device=kv.device).view(B, 1, 1)

    def one(ql, qp, ib, kv, k_pe):
        valid = ib >= 0
        ii = ib.clamp_min(0)
        kvs = kv[bi, ii].float()                                            # [B, tb, K, dl]
        kps = k_pe[bi, ii].float()                                          # [B, tb, K, dr]
        s = (torch.einsum("bthd,btkd->bthk", ql.float(), kvs) + torch.einsum("bthd,btkd->bthk", qp.float(), kps)) * softmax_scale
        p = _softmax_selected(s, valid.unsqueeze(2))                        # [B, tb, H, K]
        o = torch.einsum("bthk,btkd->bthd", p, kvs).to(ql.dtype)
        return o, p.mean(dim=2)

    return _blocks(one, q_lat.shape[1], block, recompute, q_lat, q_pe, idx, shared=(kv, k_pe))


def selected_kl_loss(scores, idx, p_target, reduction: str = "mean"):
    """KL(p_target || softmax over the selected keys of the indexer scores).

    scores [B, T, S] (the indexer's, -inf where a key is not visible); idx [B, T, K]; p_target [B, T, K] (detached here).
    ``reduction``: "mean" (alias "batchmean") averages the per-query divergences over query tokens, "sum" adds them."""
    valid = idx >= 0
    sc = torch.gather(scores, 2, idx.clamp_min(0)).masked_fill(~valid, float("-inf"))
    m = sc.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    z = sc - m
    logq = z - torch.log(torch.exp(z).sum(dim=-1, keepdim=True).clamp_min(1e-30))
    tgt = p_target.detach().float()
    tgt = tgt / tgt.sum(dim=-1, keepdim=True).clamp_min(1e-30)
    kl = torch.where((tgt > 0) & valid, tgt * (torch.log(tgt.clamp_min(1e-30)) - logq), torch.zeros_like(tgt))
    tot = kl.sum()
    if reduction == "sum":
        return tot
    if reduction in ("mean", "batchmean"):
        return tot / (kl.shape[0] * kl.shape[1])
    raise ValueError(f"unknown KL reduction {reduction!r}")
