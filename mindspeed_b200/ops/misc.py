"""Front ends of csrc/kernels/misc_ops.cu with eager fallbacks (CPU path and oracles)."""
from __future__ import annotations

import ctypes

import torch

from . import loader
from ._dtypes import code


def scaled_masked_softmax_ref(x, mask, scale, causal=False):
    s = x.float() * scale
    if mask is not None:
        s = s.masked_fill(mask.bool(), float("-inf"))
    if causal:
        sq, sk = x.shape[-2], x.shape[-1]
        i = torch.arange(sq, device=x.device).view(-1, 1) + (sk - sq)
        j = torch.arange(sk, device=x.device).view(1, -1)
        s = s.masked_fill(j > i, float("-inf"))
    return torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0).to(x.dtype)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale, causal):
        L = loader.require_lib()
        xc = x.contiguous()
        cols, sq = xc.shape[-1], xc.shape[-2]
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        m = None
        mask_rows = 1
        if mask is not None:
            m = mask.to(torch.uint8).expand(*([1] * (xc.dim() - mask.dim())), *mask.shape) if mask.dim() < xc.dim() else mask.to(torch.uint8)
            # broadcast over heads: mask [b,1,sq,sk] with x [b,n,sq,sk] is handled by expanding (rare path, small)
            m = m.expand_as(xc).contiguous()
            mask_rows = rows
        loader.check(L.msb_scaled_masked_softmax_fwd(loader.p(xc), loader.p(m), loader.p(y), ctypes.c_longlong(rows), cols,
                                                     ctypes.c_float(scale), sq, int(causal), ctypes.c_longlong(mask_rows), code(x.dtype),
                                                     ctypes.c_void_p(loader.stream_ptr())), "softmax_fwd")
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        L = loader.require_lib()
        (y,) = ctx.saved_tensors
        dy = dy.contiguous()
        cols = y.shape[-1]
        dx = torch.empty_like(y)
        loader.check(L.msb_scaled_masked_softmax_bwd(loader.p(dy), loader.p(y), loader.p(dx), ctypes.c_longlong(y.numel() // cols), cols,
                                                     ctypes.c_float(ctx.scale), code(y.dtype), ctypes.c_void_p(loader.stream_ptr())),
                     "softmax_bwd")
        return dx, None, None, None


def scaled_masked_softmax(x, mask=None, scale=1.0, causal=False):
    if x.is_cuda and loader.use_kernels(x):
        return _SoftmaxFn.apply(x, mask, float(scale), bool(causal))
    return scaled_masked_softmax_ref(x, mask, scale, causal)


def ring_attention_update_ref(prev_out, prev_max, prev_sum, cur_out, cur_max, cur_sum):
    """out [rows, d]; max / sum [rows] (reference math: mindspeed/core/context_parallel/utils.py:77-119)."""
    m = torch.maximum(prev_max, cur_max)
    a, b = prev_sum * torch.exp(prev_max - m), cur_sum * torch.exp(cur_max - m)
    l = a + b
    out = prev_out.float() * (a / l).unsqueeze(-1) + cur_out.float() * (b / l).unsqueeze(-1)
    return out.to(prev_out.dtype), m, l


def ring_attention_update(prev_out, prev_max, prev_sum, cur_out, cur_max, cur_sum):
    if not (prev_out.is_cuda and loader.use_kernels(prev_out)):
        return ring_attention_update_ref(prev_out, prev_max, prev_sum, cur_out, cur_max, cur_sum)
    L = loader.require_lib()
    d = prev_out.shape[-1]
    rows = prev_out.numel() // d
    out = torch.empty_like(prev_out)
    om, os_ = torch.empty_like(prev_max), torch.empty_like(prev_sum)
    loader.check(L.msb_ring_attention_update(loader.p(prev_out.contiguous()), loader.p(prev_max.contiguous()), loader.p(prev_sum.contiguous()),
                                             loader.p(cur_out.contiguous()), loader.p(cur_max.contiguous()), loader.p(cur_sum.contiguous()),
                                             loader.p(out), loader.p(om), loader.p(os_), ctypes.c_longlong(rows), d, code(prev_out.dtype),
                                             ctypes.c_void_p(loader.stream_ptr())), "ring_attention_update")
    return out, om, os_


def add_rmsnorm(x, residual, gamma, eps=1e-5):
    """(h, y) with h = x + residual and y = rmsnorm(h) * gamma (forward only; used by inference-style fused paths)."""
    if not (x.is_cuda and loader.use_kernels(x)):
        h = x + residual
        hf = h.float()
        return h, (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)
    L = loader.require_lib()
    cols = x.shape[-1]
    h, y = torch.empty_like(x), torch.empty_like(x)
    loader.check(L.msb_add_rmsnorm(loader.p(x.contiguous()), loader.p(residual.contiguous()), loader.p(gamma), loader.p(h), loader.p(y), None,
                                   ctypes.c_longlong(x.numel() // cols), cols, ctypes.c_float(eps), code(x.dtype),
                                   ctypes.c_void_p(loader.stream_ptr())), "add_rmsnorm")
    return h, y


def quant_1x128(x, pow2=False):
    """Kernel form of ``ops.quant.quant_1x128`` (e4m3)."""
    if not (x.is_cuda and loader.use_kernels(x)):
        from .quant import quant_1x128 as ref
        return ref(x, pow2=pow2)
    L = loader.require_lib()
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    loader.check(L.msb_quant_1x128(loader.p(x.contiguous()), loader.p(q), loader.p(sc), ctypes.c_longlong(M), K, int(pow2), code(x.dtype),
                                   ctypes.c_void_p(loader.stream_ptr())), "quant_1x128")
    return q, sc
