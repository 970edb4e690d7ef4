"""RMSNorm (and the eager LayerNorm wrapper).

``rms_norm(x, weight, eps)`` is an autograd function over csrc/kernels/norm.cu on a GPU and
the eager restatement on CPU (reference semantics: mindspeed/core/fusions/fused_rms_norm.py:7-42).
"""
from __future__ import annotations

import ctypes

import torch

from . import loader
from ._dtypes import code


def rms_norm_ref(x, weight, eps=1e-5, zero_centered=False):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float() + 1.0 if zero_centered else weight.float()
    return (xf * rstd * w).to(x.dtype)


_scratch = {}


def _get_scratch(dev, elems):
    buf = _scratch.get(dev)
    if buf is None or buf.numel() < elems:
        buf = torch.empty(elems, dtype=torch.float32, device=dev)
        _scratch[dev] = buf
    return buf


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, zero_centered):
        L = loader.require_lib()
        xc = x.contiguous()
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        loader.check(L.msb_rmsnorm_fwd(loader.p(xc), loader.p(weight), loader.p(y), loader.p(rstd), rows, cols,
                                       ctypes.c_float(eps), int(zero_centered), code(x.dtype),
                                       ctypes.c_void_p(loader.stream_ptr())), "rmsnorm_fwd")
        ctx.save_for_backward(xc, weight, rstd)
        ctx.zero_centered = zero_centered
        return y

    @staticmethod
    def backward(ctx, dy):
        L = loader.require_lib()
        x, weight, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        cols = x.shape[-1]
        rows = x.numel() // cols
        dx = torch.empty_like(x)
        dw = torch.empty_like(weight)
        L.msb_rmsnorm_bwd_scratch_elems.restype = ctypes.c_size_t
        scratch = _get_scratch(x.device, L.msb_rmsnorm_bwd_scratch_elems(rows, cols))
        loader.check(L.msb_rmsnorm_bwd(loader.p(dy), loader.p(x), loader.p(weight), loader.p(rstd), loader.p(dx),
                                       loader.p(dw), loader.p(scratch), rows, cols, int(ctx.zero_centered), 0,
                                       code(x.dtype), ctypes.c_void_p(loader.stream_ptr())), "rmsnorm_bwd")
        return dx, dw, None, None


class _AddRMSNormFn(torch.autograd.Function):
    """(h, y) = (x + residual, rmsnorm(x + residual) * weight) in one pass over the row; the backward adds the
    gradient that reaches h directly to the one that comes back through the norm inside the same kernel
    (reference: the residual-add + norm fusion of mindspeed/ops/csrc/cann/npu_dropout_add_layer_norm.cpp, RMSNorm form)."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps, zero_centered):
        L = loader.require_lib()
        xc, rc = x.contiguous(), residual.contiguous()
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        h, y = torch.empty_like(xc), torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        loader.check(L.msb_add_rmsnorm_fwd(loader.p(xc), loader.p(rc), loader.p(weight), loader.p(h), loader.p(y), loader.p(rstd),
                                           rows, cols, ctypes.c_float(eps), int(zero_centered), code(x.dtype),
                                           ctypes.c_void_p(loader.stream_ptr())), "add_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.zero_centered = zero_centered
        ctx.mark_non_differentiable(rstd)
        return h, y

    @staticmethod
    def backward(ctx, dh, dy):
        L = loader.require_lib()
        h, weight, rstd = ctx.saved_tensors
        cols = h.shape[-1]
        rows = h.numel() // cols
        dw = torch.empty_like(weight)
        if dy is None:
            return dh, dh, torch.zeros_like(weight), None, None
        dx = torch.empty_like(h)
        L.msb_rmsnorm_bwd_scratch_elems.restype = ctypes.c_size_t
        scratch = _get_scratch(h.device, L.msb_rmsnorm_bwd_scratch_elems(rows, cols))
        loader.check(L.msb_rmsnorm_bwd_add(loader.p(dy.contiguous()), loader.p(h), loader.p(weight), loader.p(rstd), loader.p(dx),
                                           loader.p(dw), loader.p(scratch), rows, cols, int(ctx.zero_centered), 0, code(h.dtype),
                                           loader.p(dh.contiguous()) if dh is not None else None,
                                           ctypes.c_void_p(loader.stream_ptr())), "rmsnorm_bwd_add")
        return dx, dx, dw, None, None


def add_rms_norm(x, residual, weight, eps=1e-5, zero_centered=False, fused=True):
    """Returns (h, y) with h = x + residual and y = rmsnorm(h) * weight."""
    if (fused and x.is_cuda and loader.use_kernels(x) and weight.dtype == x.dtype and residual.dtype == x.dtype
            and x.shape == residual.shape and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384):
        return _AddRMSNormFn.apply(x, residual, weight, eps, zero_centered)
    h = x + residual
    return h, rms_norm(h, weight, eps, zero_centered, fused)


def rms_norm(x, weight, eps=1e-5, zero_centered=False, fused=True):
    if fused and x.is_cuda and loader.use_kernels(x) and weight.dtype == x.dtype:
        return _RMSNormFn.apply(x, weight, eps, zero_centered)
    return rms_norm_ref(x, weight, eps, zero_centered)


def dropout_add_norm(x0, residual, weight, bias, dropout_p, epsilon, rowscale=None, layerscale=None, prenorm=False,
                     residual_in_fp32=False, return_dropout_mask=False, is_rms_norm=False, training=True):
    """out = norm(dropout(x0 * rowscale * layerscale) + residual) * weight (+ bias).

    ``rowscale`` [batch, seq] scales whole token rows (stochastic depth), ``layerscale`` [hidden] scales channels, both
    before the dropout; ``prenorm`` also returns the un-normalised sum (the next residual stream, in fp32 when
    ``residual_in_fp32``); ``return_dropout_mask`` appends the keep mask.  Without dropout and scales the RMSNorm form on a
    GPU is the one-pass add + norm kernel (``add_rms_norm``); every other combination is composed from PyTorch ops.
    reference: mindspeed/ops/dropout_add_layer_norm.py:8-76, mindspeed/ops/dropout_add_rms_norm.py (same arguments;
    mindspeed/ops/csrc/cann/npu_dropout_add_layer_norm.cpp)."""
    h = x0
    if rowscale is not None:
        h = h * rowscale.reshape(*x0.shape[:-1], 1).to(h.dtype)
    if layerscale is not None:
        h = h * layerscale.reshape(*([1] * (x0.dim() - 1)), -1).to(h.dtype)
    mask = None
    p = float(dropout_p) if training else 0.0
    if p > 0.0:
        mask = torch.rand_like(h, dtype=torch.float32) >= p
        h = h * mask.to(h.dtype) / (1.0 - p)
    plain = p == 0.0 and rowscale is None and layerscale is None
    if (plain and is_rms_norm and residual is not None and bias is None and h.is_cuda and not residual_in_fp32
            and h.dtype == residual.dtype and loader.lib() is not None):
        pre, out = add_rms_norm(h, residual, weight, epsilon)
    else:
        pre = h if residual is None else (h.float() + residual.float() if residual_in_fp32 else h + residual.to(h.dtype))
        if is_rms_norm:
            out = rms_norm_ref(pre.to(x0.dtype), weight, epsilon)
        else:
            out = torch.nn.functional.layer_norm(pre.to(x0.dtype), (x0.shape[-1],), weight, None, epsilon)
        if bias is not None:
            out = out + bias
    ret = (out, pre) if prenorm else (out,)
    if return_dropout_mask:
        ret = ret + (mask if mask is not None else torch.ones_like(x0, dtype=torch.bool),)
    return ret[0] if len(ret) == 1 else ret


def dropout_add_layer_norm(x0, residual, weight, bias, dropout_p, epsilon, rowscale=None, layerscale=None, prenorm=False,
                           residual_in_fp32=False, return_dropout_mask=False, training=True):
    return dropout_add_norm(x0, residual, weight, bias, dropout_p, epsilon, rowscale, layerscale, prenorm, residual_in_fp32,
                            return_dropout_mask, False, training)


def dropout_add_rms_norm(x0, residual, weight, bias, dropout_p, epsilon, rowscale=None, layerscale=None, prenorm=False,
                         residual_in_fp32=False, return_dropout_mask=False, training=True):
    return dropout_add_norm(x0, residual, weight, bias, dropout_p, epsilon, rowscale, layerscale, prenorm, residual_in_fp32,
                            return_dropout_mask, True, training)

