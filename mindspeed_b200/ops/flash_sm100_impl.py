"""Autograd wrapper of the tcgen05 flash-attention forward (csrc/kernels/flash_attn_sm100.cu).

Forward and backward are the hand-written kernels of csrc/kernels/flash2_sm100.cu; the LSE convention (natural log of
the softmax denominator of the scaled scores) is the one ring attention and the reference implementation use, so blocks
computed here can be merged with or differentiated against a global LSE.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import gemm as G
from . import loader

def flash_fwd(q, k, v, causal, scale, q_offset=None, kernel=2):
    """q [sq,b,nq,128], k/v [sk,b,nkv,128] bf16 (strided views allowed) -> (o [sq,b,nq,128], lse [b,nq,sq] fp32).
    ``kernel`` 2 = two query tiles per CTA with P in tensor memory (default), 1 = the single-tile kernel."""
    L = loader.require_lib()
    fn = L.msb_flash_fwd2 if kernel == 2 else L.msb_flash_fwd
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
    loader.check(fn(loader.p(q), loader.p(k), loader.p(v), loader.p(o), loader.p(lse), sq, sk, b, nq, nkv,
                                 ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
                                 ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)), int(causal), int(q_offset),
                                 ctypes.c_float(scale), loader.p(st), ctypes.c_void_p(loader.stream_ptr())), "flash_fwd")
    return o, lse


def flash_bwd(dout, q, k, v, o, lse, causal, scale, q_offset=None):
    """Gradients (dq, dk, dv) on the tcgen05 backward kernel.  Shapes as ``flash_fwd``; ``o`` contiguous, ``lse`` the
    forward's (or, for ring attention, the global) log-sum-exp.  dQ is accumulated in fp32 by the key tiles (TMA
    reduce-adds, so its low bits can differ between runs) and rounded to bf16 once at the end."""
    L = loader.require_lib()
    sq, b, nq, d = q.shape
    sk, nkv = k.shape[0], k.shape[2]
    if q_offset is None:
        q_offset = sk - sq if causal else 0
    if dout.stride(-1) != 1 or any((st * 2) % 16 for st in dout.stride()[:-1]) or dout.data_ptr() % 16:
        dout = dout.contiguous()
    o = o if o.is_contiguous() else o.contiguous()
    lse = lse if lse.is_contiguous() else lse.contiguous()
    dev = q.device
    sq_pad = (sq + 127) // 128 * 128
    dq32 = torch.zeros(sq, b, nq, d, dtype=torch.float32, device=dev)
    never_seen = causal and (sq + q_offset < sk)       # trailing key tiles that no query row reaches keep zero gradients
    # few (key tile, KV head) pairs would leave most SMs idle: then one CTA per QUERY head, partial dK / dV summed in fp32
    n_ctas = ((sk + 127) // 128) * nkv * b
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    split = nq > nkv and n_ctas < 2 * sms
    if split:
        dk = torch.zeros(sk, b, nkv, d, dtype=torch.float32, device=dev)
        dv = torch.zeros(sk, b, nkv, d, dtype=torch.float32, device=dev)
    else:
        alloc = torch.zeros if never_seen else torch.empty
        dk = alloc(sk, b, nkv, d, dtype=torch.bfloat16, device=dev)
        dv = alloc(sk, b, nkv, d, dtype=torch.bfloat16, device=dev)
    stats = torch.empty(2, b, nq, sq_pad, dtype=torch.float32, device=dev)
    ll = ctypes.c_longlong
    st = G.status_word(dev)
    loader.check(L.msb_flash_bwd(loader.p(q), loader.p(k), loader.p(v), loader.p(o), loader.p(dout), loader.p(lse), loader.p(dq32),
                                 loader.p(dk), loader.p(dv), loader.p(stats[0]), loader.p(stats[1]), int(split), sq, sk, b, nq, nkv,
                                 ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
                                 ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)), ll(dout.stride(0)), ll(dout.stride(1)),
                                 ll(dout.stride(2)), int(causal), int(q_offset), ctypes.c_float(scale), loader.p(st),
                                 ctypes.c_void_p(loader.stream_ptr())), "flash_bwd")
    if split:
        dk, dv = dk.to(torch.bfloat16), dv.to(torch.bfloat16)
    return dq32.to(torch.bfloat16), dk, dv


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
        dq, dk, dv = flash_bwd(do, q, k, v, o, lse, causal, scale)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, causal, softmax_scale, return_lse):
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    o, lse = _FlashFn.apply(q, k, v, bool(causal), float(scale))
    return (o, lse) if return_lse else o
