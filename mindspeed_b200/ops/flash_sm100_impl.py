"""Autograd wrapper of the tcgen05 flash-attention forward (csrc/kernels/flash_attn_sm100.cu).

Forward: hand-written kernel producing O and the per-row log-sum-exp.  Backward: until the sm_100a backward kernel
lands, the flash backward of the framework library is driven with this kernel's O and LSE (they use the same
convention: natural-log LSE of the scaled scores), so the two halves are interchangeable.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import gemm as G
from . import loader

_RNG = {}


def _rng_template(dev):
    """Placeholder rng-state tensors of the right type for the library backward (dropout is 0, so they are unused)."""
    t = _RNG.get(dev)
    if t is None:
        q = torch.zeros(1, 1, 16, 64, device=dev, dtype=torch.bfloat16)
        res = torch.ops.aten._scaled_dot_product_flash_attention(q, q, q, 0.0, False, False)
        t = (res[6], res[7])
        _RNG[dev] = t
    return t


def flash_fwd(q, k, v, causal, scale, q_offset=None):
    """q [sq,b,nq,128], k/v [sk,b,nkv,128] bf16 (strided views allowed) -> (o [sq,b,nq,128], lse [b,nq,sq] fp32)."""
    L = loader.require_lib()
    sq, b, nq, d = q.shape
    sk, nkv = k.shape[0], k.shape[2]
    for t in (q, k, v):
        if t.stride(-1) != 1 or any((s * 2) % 16 for s in t.stride()[:-1]) or t.data_ptr() % 16:
            raise ValueError("flash_fwd: operands need a contiguous last dim and 16-byte aligned strides")
    o = torch.empty(sq, b, nq, d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, nq, sq, dtype=torch.float32, device=q.device)
    if q_offset is None:
        q_offset = sk - sq if causal else 0
    ll = ctypes.c_longlong
    st = G.status_word(q.device)
    loader.check(L.msb_flash_fwd(loader.p(q), loader.p(k), loader.p(v), loader.p(o), loader.p(lse), sq, sk, b, nq, nkv,
                                 ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
                                 ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)), int(causal), int(q_offset),
                                 ctypes.c_float(scale), loader.p(st), ctypes.c_void_p(loader.stream_ptr())), "flash_fwd")
    return o, lse


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, scale)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        sq, b, nq, d = q.shape
        sk, nkv = k.shape[0], k.shape[2]
        rep = nq // nkv
        qb, kb, vb = q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3)
        if rep > 1:
            kb, vb = kb.repeat_interleave(rep, 1), vb.repeat_interleave(rep, 1)
        seed, off = _rng_template(q.device)
        dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            do.permute(1, 2, 0, 3), qb, kb, vb, o.permute(1, 2, 0, 3), lse, None, None, sq, sk, 0.0, causal, seed, off, scale=scale)
        if rep > 1:
            dk = dk.reshape(b, nkv, rep, sk, d).sum(2)
            dv = dv.reshape(b, nkv, rep, sk, d).sum(2)
        return dq.permute(2, 0, 1, 3), dk.permute(2, 0, 1, 3), dv.permute(2, 0, 1, 3), None, None


def flash_attention(q, k, v, causal, softmax_scale, return_lse):
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    o, lse = _FlashFn.apply(q, k, v, bool(causal), float(scale))
    return (o, lse) if return_lse else o
