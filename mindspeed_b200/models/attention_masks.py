"""Attention mask and position utilities.

  alibi_slopes / alibi_bias            ALiBi head slopes (powers of 2^(-8/n), with the interleave rule for head counts that
                                       are not powers of two) and the additive bias, sharded over tensor-parallel ranks
  compressed_causal_mask               the fixed 2048 x 2048 lower-triangular mask attention kernels accept as a compressed
                                       stand-in for an S x S causal mask (sparse_mode 2/3/4 of the reference's FA call)
  eod_reset                            packed-sequence handling: from token ids and the end-of-document id derive
                                       per-document position ids, cumulative sequence lengths (THD layout), the loss mask
                                       and - when an explicit mask is wanted - the block-diagonal causal mask
reference: mindspeed/core/transformer/flash_attention/alibi/*, generate_mask/generate_mask.py:16-71,
reset_attention_mask/adaptor.py:218-759.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch


def alibi_slopes(num_heads: int) -> torch.Tensor:
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(num_heads).is_integer():
        return torch.tensor(pow2(num_heads))
    closest = 2 ** math.floor(math.log2(num_heads))
    extra = pow2(2 * closest)[0::2][:num_heads - closest]
    return torch.tensor(pow2(closest) + extra)


def alibi_bias(num_heads: int, seq_q: int, seq_k: int, tp_rank: int = 0, tp_size: int = 1, dtype=torch.float32, device=None,
               symmetric: bool = False) -> torch.Tensor:
    """[heads_local, seq_q, seq_k]; bias = -slope * (i - j) for j <= i (or |i - j| when ``symmetric``)."""
    slopes = alibi_slopes(num_heads).to(device=device)
    per = num_heads // tp_size
    slopes = slopes[tp_rank * per:(tp_rank + 1) * per]
    i = torch.arange(seq_q, device=device).unsqueeze(1) + (seq_k - seq_q)
    j = torch.arange(seq_k, device=device).unsqueeze(0)
    dist = (i - j).abs() if symmetric else (i - j).clamp(min=0)
    return (-slopes.view(-1, 1, 1) * dist.unsqueeze(0)).to(dtype)


_COMPRESSED = {}


def compressed_causal_mask(device=None, size: int = 2048) -> torch.Tensor:
    """True = masked.  Cached per device."""
    key = (str(device), size)
    if key not in _COMPRESSED:
        _COMPRESSED[key] = torch.triu(torch.ones(size, size, dtype=torch.bool, device=device), diagonal=1)
    return _COMPRESSED[key]


def eod_reset(tokens: torch.Tensor, eod_token: int, reset_position_ids: bool = True, reset_attention_mask: bool = True,
              eod_mask_loss: bool = True, build_dense_mask: bool = False) -> Dict[str, Optional[torch.Tensor]]:
    """tokens [B, S].  Documents end AT their eod token (the eod belongs to the document it closes)."""
    B, S = tokens.shape
    dev = tokens.device
    is_eod = tokens == eod_token
    pos = torch.arange(S, device=dev).unsqueeze(0).expand(B, S).clone()
    doc_id = torch.zeros(B, S, dtype=torch.long, device=dev)
    if reset_position_ids or reset_attention_mask:
        starts = torch.zeros(B, S, dtype=torch.bool, device=dev)
        starts[:, 0] = True
        starts[:, 1:] = is_eod[:, :-1]
        doc_id = torch.cumsum(starts.long(), dim=1) - 1
        if reset_position_ids:
            start_pos = torch.where(starts, pos, torch.zeros_like(pos))
            start_pos = torch.cummax(start_pos, dim=1).values
            pos = pos - start_pos
    loss_mask = torch.ones(B, S, dtype=torch.float32, device=dev)
    if eod_mask_loss:
        loss_mask[is_eod] = 0.0
    cu = None
    if reset_attention_mask:
        # THD: all batch rows concatenated; boundaries wherever a document (or a row) starts
        flat_start = torch.zeros(B * S, dtype=torch.bool, device=dev)
        flat_start[0::S] = True
        flat_start |= torch.cat([torch.zeros(B, 1, dtype=torch.bool, device=dev), is_eod[:, :-1]], dim=1).reshape(-1)
        idx = torch.nonzero(flat_start, as_tuple=False).squeeze(1)
        cu = torch.cat([idx, torch.tensor([B * S], device=dev)]).to(torch.int32)
    dense = None
    if build_dense_mask:
        causal = torch.tril(torch.ones(S, S, dtype=torch.bool, device=dev))
        same = doc_id.unsqueeze(2) == doc_id.unsqueeze(1) if reset_attention_mask else torch.ones(B, S, S, dtype=torch.bool, device=dev)
        dense = ~(causal.unsqueeze(0) & same)            # True = masked
        dense = dense.unsqueeze(1)
    return {"position_ids": pos, "loss_mask": loss_mask, "cu_seqlens": cu, "attention_mask": dense, "document_ids": doc_id,
            "max_seqlen": int((cu[1:] - cu[:-1]).max()) if cu is not None else S}
