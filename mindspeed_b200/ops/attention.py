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


# ---------------------------------------------------------------------------------------------------------
# Block primitives for ring / KV-allgather attention: forward returning LSE, backward taking the GLOBAL output
# and LSE (so partial blocks of one softmax row can be differentiated independently).
# ---------------------------------------------------------------------------------------------------------
def attn_bwd_ref(dout, q, k, v, out, lse, causal, softmax_scale=None, q_offset=0):
    """fp32 reference backward. Shapes as the forward; lse [b, n, sq] is the global log-sum-exp of each row."""
    sq, b, nq, d = q.shape
    sk, nkv = k.shape[0], k.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    rep = nq // nkv
    qf = q.permute(1, 2, 0, 3).float()
    kf = k.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
    vf = v.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
    do = dout.permute(1, 2, 0, 3).float()
    of = out.permute(1, 2, 0, 3).float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(sq, device=q.device).view(sq, 1) + q_offset
        kj = torch.arange(sk, device=q.device).view(1, sk)
        s = s.masked_fill((kj > qi).view(1, 1, sq, sk), float("-inf"))
    p = torch.exp(s - lse.float().unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0, posinf=0.0)
    dv = torch.matmul(p.transpose(-1, -2), do)
    dp = torch.matmul(do, vf.transpose(-1, -2))
    delta = (do * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    if rep > 1:
        dk = dk.view(b, nkv, rep, sk, -1).sum(2)
        dv = dv.view(b, nkv, rep, sk, -1).sum(2)
    back = lambda t, ref: t.permute(2, 0, 1, 3).contiguous().to(ref.dtype)
    return back(dq, q), back(dk, k), back(dv, v)


def attn_fwd_block(q, k, v, causal, softmax_scale=None):
    """(out [sq,b,nq,dv], lse [b,nq,sq] fp32, ctx) for one (Q block, KV block) pair; causal = top-left aligned."""
    if q.is_cuda and get_backend(q) == "sm100":
        from . import flash_sm100
        if flash_sm100.supports(q, k, v, causal):
            from .flash_sm100_impl import flash_fwd
            scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
            out, lse = flash_fwd(q, k, v, causal, scale, q_offset=0)
            return out, lse, "sm100"
    if q.is_cuda and get_backend(q) != "ref":
        sq, b, nq, d = q.shape
        nkv = k.shape[2]
        rep = nq // nkv
        qb = q.permute(1, 2, 0, 3)
        kb = k.permute(1, 2, 0, 3)
        vb = v.permute(1, 2, 0, 3)
        if rep > 1:
            kb, vb = kb.repeat_interleave(rep, 1), vb.repeat_interleave(rep, 1)
        res = torch.ops.aten._scaled_dot_product_flash_attention(qb, kb, vb, 0.0, causal, False, scale=softmax_scale)
        out, lse = res[0], res[1]
        ctx = (res[6], res[7])  # philox seed / offset
        return out.permute(2, 0, 1, 3), lse, ctx
    out, lse = attention_ref(q, k, v, causal, softmax_scale, return_lse=True)
    return out, lse, None


def attn_bwd_block(dout, q, k, v, out, lse, causal, softmax_scale=None, ctx=None):
    if isinstance(ctx, str) and ctx == "sm100":
        from .flash_sm100_impl import flash_bwd
        scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
        return flash_bwd(dout, q, k, v, out, lse, causal, scale, q_offset=0)
    if q.is_cuda and get_backend(q) != "ref" and ctx is not None:
        sq, b, nq, d = q.shape
        sk, nkv = k.shape[0], k.shape[2]
        rep = nq // nkv
        qb, kb, vb = q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3)
        if rep > 1:
            kb, vb = kb.repeat_interleave(rep, 1), vb.repeat_interleave(rep, 1)
        dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            dout.permute(1, 2, 0, 3), qb, kb, vb, out.permute(1, 2, 0, 3), lse.contiguous(), None, None, sq, sk, 0.0, causal,
            ctx[0], ctx[1], scale=softmax_scale)
        if rep > 1:
            dk = dk.view(b, nkv, rep, sk, -1).sum(2)
            dv = dv.view(b, nkv, rep, sk, -1).sum(2)
        return dq.permute(2, 0, 1, 3), dk.permute(2, 0, 1, 3), dv.permute(2, 0, 1, 3)
    return attn_bwd_ref(dout, q, k, v, out, lse, causal, softmax_scale)


def merge_lse(out1, lse1, out2, lse2):
    """Online-softmax merge of two partial attention results over disjoint key sets
    (reference math: mindspeed/core/context_parallel/utils.py:77-119; here in LSE form).
    out [s,b,n,d]; lse [b,n,s]."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).permute(2, 0, 1).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).permute(2, 0, 1).unsqueeze(-1)
    out = out1.float() * w1 + out2.float() * w2
    return out.to(out1.dtype), lse


def varlen_attention(q, k, v, cu_seqlens, causal=True, softmax_scale=None, backend=None):
    """Attention over packed sequences: q / k / v [s, b, n, d] hold several documents back to back, ``cu_seqlens`` (host
    integers, first 0, last s) their boundaries, the same for every batch row (b = 1 when they come from the data);
    every document attends only to itself.  One attention call per document on the configured backend (the tcgen05
    kernels on a GPU), so the cost is the sum of the documents' squares instead of s^2; documents of one common length
    are folded into the batch axis and take a single call.
    reference semantics: actual_seq_qlen / actual_seq_kvlen of npu_fusion_attention in the TND layout
    (mindspeed/ops/fusion_attention_v2.py:22-114) as used by the reset-attention-mask path
    (mindspeed/core/transformer/flash_attention/reset_attention_mask/adaptor.py:218-759)."""
    bounds = [int(x) for x in cu_seqlens]
    if bounds[0] != 0 or bounds[-1] != q.shape[0]:
        raise ValueError(f"cu_seqlens must run from 0 to the sequence length {q.shape[0]}, got {bounds[0]}..{bounds[-1]}")
    lens = {b - a for a, b in zip(bounds[:-1], bounds[1:])}
    if len(lens) == 1 and len(bounds) > 2:
        # equal sub-sequences: fold them into the batch axis, one attention call for all of them
        L, m = lens.pop(), len(bounds) - 1
        s, b = q.shape[0], q.shape[1]

        def fold(x):
            return x.reshape(m, L, b, x.shape[2], x.shape[3]).transpose(0, 1).reshape(L, m * b, x.shape[2], x.shape[3])
        o = flash_attention(fold(q), fold(k), fold(v), causal=causal, softmax_scale=softmax_scale, backend=backend)
        return o.reshape(L, m, b, o.shape[2], o.shape[3]).transpose(0, 1).reshape(s, b, o.shape[2], o.shape[3])
    outs = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b > a:
            outs.append(flash_attention(q[a:b], k[a:b], v[a:b], causal=causal, softmax_scale=softmax_scale, backend=backend))
    return torch.cat(outs, dim=0)


def alibi_attention(q, k, v, slopes, causal=True, softmax_scale=None, mode=0, signed=False, block=1024):
    """Attention with the ALiBi position bias evaluated from the per-head ``slopes [n]`` (no [n, s, s] bias tensor is built).

    q [sq, b, n, d]; k, v [sk, b, nkv, d].  ``mode`` 0 / 2: bias = -slope * |i - j| (0 is the reference's dense-bias form,
    2 its in-kernel form: the same values); 3: -slope * sqrt|i - j|.  ``signed`` (the reference's diagonal-opposite option,
    modes 0 / 2): bias = slope * (j - i), negative for past keys and positive for future ones - the same as the default under
    a causal mask.  Query rows are processed in blocks, each re-computed in backward, so one block's [b, n, tb, sk]
    scores are the largest temporary.  fp32 math.
    reference: mindspeed/core/transformer/flash_attention/alibi/alibi.py:28-124, dot_product_attention.py:19-106."""
    from torch.utils.checkpoint import checkpoint
    sq, b, nq, d = q.shape
    sk, nkv = k.shape[0], k.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    rep = nq // nkv
    off = sk - sq
    sl = slopes.float().view(1, nq, 1, 1)

    def one(qb, k, v, t0):
        tb = qb.shape[0]
        kf = k.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
        vf = v.permute(1, 2, 0, 3).float().repeat_interleave(rep, dim=1)
        s = torch.matmul(qb.permute(1, 2, 0, 3).float(), kf.transpose(-1, -2)) * scale
        qi = torch.arange(t0, t0 + tb, device=q.device).view(tb, 1) + off
        kj = torch.arange(sk, device=q.device).view(1, sk)
        rel = (kj - qi).float()
        if mode == 3:
            bias = -sl * rel.abs().sqrt().view(1, 1, tb, sk)
        elif signed:
            bias = sl * rel.view(1, 1, tb, sk)
        else:
            bias = -sl * rel.abs().view(1, 1, tb, sk)
        s = s + bias
        if causal:
            s = s.masked_fill((kj > qi).view(1, 1, tb, sk), float("-inf"))
        p = torch.softmax(s, dim=-1)
        return torch.matmul(p, vf).permute(2, 0, 1, 3).to(q.dtype)

    outs = []
    need = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    for t0 in range(0, sq, block):
        qb = q[t0:t0 + block]
        outs.append(checkpoint(one, qb, k, v, t0, use_reentrant=False) if need and sq > block else one(qb, k, v, t0))
    return torch.cat(outs, dim=0).contiguous()


def band_attention(q, k, v, pre: int, nxt: int, softmax_scale=None, block: int = 512):
    """Sliding-window attention: query i (bottom-right aligned when sk > sq) sees keys j with i - pre <= j <= i + nxt.

    q [sq, b, n, d]; k, v [sk, b, nkv, d].  Query rows are taken ``block`` at a time and only the keys a block can see are
    sliced out, so the work is O(s * (pre + nxt + block)) instead of O(s^2); every block is re-computed in backward.
    fp32 math.  The window bounds of the reference's attention op: ``pre_tockens`` / ``next_tockens`` with ``sparse_mode`` 0 / 4
    (mindspeed/ops/fusion_attention_v2.py:22-114)."""
    from torch.utils.checkpoint import checkpoint
    sq, sk = q.shape[0], k.shape[0]
    off = sk - sq
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])

    def one(qb, kb, vb, t0, lo):
        tb, kb_n = qb.shape[0], kb.shape[0]
        qi = torch.arange(t0, t0 + tb, device=q.device).view(tb, 1) + off
        kj = torch.arange(lo, lo + kb_n, device=q.device).view(1, kb_n)
        hidden = (kj < qi - pre) | (kj > qi + nxt)
        return attention_ref(qb, kb, vb, causal=False, softmax_scale=scale, mask=hidden.view(1, 1, tb, kb_n))

    need = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    outs = []
    for t0 in range(0, sq, block):
        t1 = min(sq, t0 + block)
        lo, hi = max(0, t0 + off - pre), min(sk, t1 - 1 + off + nxt + 1)
        if hi <= lo:                                   # no visible key: zero rows
            outs.append(q.new_zeros(t1 - t0, q.shape[1], q.shape[2], v.shape[-1]))
            continue
        args = (q[t0:t1], k[lo:hi], v[lo:hi], t0, lo)
        outs.append(checkpoint(one, *args, use_reentrant=False) if need and sq > block else one(*args))
    return torch.cat(outs, dim=0).contiguous()

