"""Lightning indexer of DeepSeek sparse attention: a cheap per-token relevance score over earlier tokens and the
top-k selection that the sparse attention then attends to.

      I[t, s] = sum_h  w[t, h] * relu( q[t, h, :] . k[s, :] )          (s <= t under the causal mask)
      index[t] = top-k over s of I[t, s]

``indexer_scores`` evaluates I in blocks of query rows so the [T, S] score matrix of one block - never of the whole
sequence times heads - is resident; ``sparse_attention_mask`` turns the selection into an additive mask.
Differentiable with respect to q, k and w (the indexer is trained with a KL loss against the dense attention
distribution).  reference: mindspeed/core/transformer/flash_attention/flash_attention/triton/triton_indexer_bf16.py:254-435,
torch_indexer_bf16.py, mindspeed/features_manager/transformer/experimental_attention_variant/dsa.py:14-22.
"""
from __future__ import annotations

import torch


def indexer_scores(q, k, w, causal: bool = True, block: int = 1024):
    """q [B, T, H, d]; k [B, S, d]; w [B, T, H] -> I [B, T, S] (fp32; -inf above the diagonal when causal)."""
    B, T, H, d = q.shape
    S = k.shape[1]
    out = []
    kt = k.transpose(1, 2)                                       # [B, d, S]
    for t0 in range(0, T, block):
        qb = q[:, t0:t0 + block]                                 # [B, tb, H, d]
        s = torch.einsum("bthd,bds->bths", qb, kt)
        sc = (torch.relu(s).float() * w[:, t0:t0 + block].float().unsqueeze(-1)).sum(dim=2)
        if causal:
            rows = torch.arange(t0, t0 + qb.shape[1], device=q.device).unsqueeze(1) + (S - T)
            cols = torch.arange(S, device=q.device).unsqueeze(0)
            sc = sc.masked_fill((cols > rows).unsqueeze(0), float("-inf"))
        out.append(sc)
    return torch.cat(out, dim=1)


def indexer_topk(q, k, w, topk: int, causal: bool = True, block: int = 1024):
    """Indices [B, T, topk] of the selected keys (padded with -1 where fewer than topk keys are visible)."""
    sc = indexer_scores(q, k, w, causal, block)
    kk = min(topk, sc.shape[-1])
    vals, idx = sc.topk(kk, dim=-1)
    idx = idx.masked_fill(torch.isinf(vals), -1)
    if kk < topk:
        idx = torch.nn.functional.pad(idx, (0, topk - kk), value=-1)
    return idx, sc


def sparse_attention_mask(idx, S: int):
    """Additive mask [B, T, S]: 0 at selected keys, -inf elsewhere."""
    B, T, _ = idx.shape
    mask = torch.full((B, T, S + 1), float("-inf"), device=idx.device)
    mask.scatter_(2, idx.clamp(min=-1).add(0).masked_fill(idx < 0, S), 0.0)
    return mask[..., :S]


def indexer_kl_loss(scores, attn_probs):
    """KL(attention || softmax(indexer scores)) averaged over tokens; ``attn_probs`` [B, T, S] is the head-summed,
    renormalised dense attention distribution (detached target)."""
    logp = torch.log_softmax(scores, dim=-1)
    tgt = attn_probs.detach().float()
    kl = torch.where(tgt > 0, tgt * (torch.log(tgt.clamp_min(1e-30)) - logp), torch.zeros_like(tgt))
    return kl.sum(-1).mean()
