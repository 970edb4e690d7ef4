"""Scaled-dot-product attention front end.

Layouts: q [sq, b, nq, d], k/v [sk, b, nkv, d] (sequence-first, GQA when nq > nkv); strided views
(for instance slices of a packed QKV activation) are accepted when the last dim is contiguous.

Back ends:
  "ref"     eager fp32 softmax(QK^T)V — CPU path and numerics oracle
  "library" torch scaled_dot_product_attention (cuDNN / flash) — optimisation level 0
  "sm100"   hand-written tcgen05 flash attention (mindspeed_b200/ops/flash_sm100.py) — level >= 1

All back ends can return the log-sum-exp per row, which ring attention needs to merge partial
results (reference: the fused attention op returns softmax max and sum separately,
mindspeed/ops/fusion_attention_v2.py:22-114; LSE = max + log(sum) carries the same information).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

_BACKEND = {"name": None}


def set_backend(name: Optional[str]):
    _BACKEND["name"] = name


def get_backend(t: torch.Tensor) -> str:
    if not t.is_cuda:
        return "ref"
    return _BACKEND["name"] or "library"


def attention_ref(q, k, v, causal=True, softmax_scale=None, mask=None, return_lse=False, q_offset=0, alibi_slopes=None):
    """fp32 reference. ``mask`` (bool, True = masked out) broadcastable to [b, n, sq, sk].
    ``q_offset``: causal mask uses absolute positions q_pos = i + q_offset (bottom-right aligned when
    q_offset = sk - sq)."""
    sq, b, nq, d = q.shape
    sk, nkv = k.shape[0], k.shape[2]
    dv = v.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    rep = nq // nkv
    qf = q.permute(1, 2, 0, 3).float()
    kf = k.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
    vf = v.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if alibi_slopes is not None:
        qi = torch.arange(sq, device=q.device).view(sq, 1) + q_offset
        kj = torch.arange(sk, device=q.device).view(1, sk)
        s = s - alibi_slopes.float().view(1, nq, 1, 1) * (qi - kj).abs().view(1, 1, sq, sk)
    if causal:
        qi = torch.arange(sq, device=q.device).view(sq, 1) + q_offset
        kj = torch.arange(sk, device=q.device).view(1, sk)
        s = s.masked_fill((kj > qi).view(1, 1, sq, sk), float("-inf"))
    if mask is not None:
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf).permute(2, 0, 1, 3).contiguous().to(q.dtype)
    if return_lse:
        return o, lse  # lse [b, n, sq]
    return o


def _library(q, k, v, causal, softmax_scale, return_lse):
    sq, b, nq, d = q.shape
    nkv = k.shape[2]
    qb, kb, vb = q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3)
    if return_lse:
        # the flash backend exposes LSE through the private op; keep the reference semantics
        out, lse = torch.ops.aten._scaled_dot_product_flash_attention(
            qb, kb.repeat_interleave(nq // nkv, 1) if nq != nkv else kb,
            vb.repeat_interleave(nq // nkv, 1) if nq != nkv else vb, 0.0, causal, False, scale=softmax_scale)[:2]
        return out.permute(2, 0, 1, 3), lse
    o = F.scaled_dot_product_attention(qb, kb, vb, is_causal=causal, scale=softmax_scale, enable_gqa=(nq != nkv))
    return o.permute(2, 0, 1, 3)


def flash_attention(q, k, v, causal=True, softmax_scale=None, return_lse=False, backend=None):
    """Returns out [sq, b, nq, dv] (and LSE [b, nq, sq] fp32 when asked)."""
    be = backend or get_backend(q)
    if be == "sm100":
        from . import flash_sm100
        if flash_sm100.supports(q, k, v, causal):
            return flash_sm100.flash_attention(q, k, v, causal, softmax_scale, return_lse)
        be = "library"
    if be == "library" and q.is_cuda:
        return _library(q, k, v, causal, softmax_scale, return_lse)
    return attention_ref(q, k, v, causal, softmax_scale, return_lse=return_lse)
