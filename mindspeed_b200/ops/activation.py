"""SwiGLU: silu(x[..., :F]) * x[..., F:]  (optionally scaled per row, for MoE experts).

reference semantics: mindspeed/core/fusions/fused_bias_swiglu.py:4-17 (torch_npu.npu_swiglu).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import loader
from ._dtypes import code


def swiglu_ref(x, row_scale=None):
    a, b = x.chunk(2, dim=-1)
    y = F.silu(a.float()) * b.float()
    if row_scale is not None:
        y = y * row_scale.float().reshape(*y.shape[:-1], 1)
    return y.to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, row_scale):
        L = loader.require_lib()
        xc = x.contiguous()
        f = xc.shape[-1] // 2
        rows = xc.numel() // (2 * f)
        y = torch.empty(*xc.shape[:-1], f, dtype=x.dtype, device=x.device)
        rs = None if row_scale is None else row_scale.float().contiguous()
        loader.check(L.msb_swiglu_fwd(loader.p(xc), loader.p(y), loader.p(rs), ctypes.c_longlong(rows), f, code(x.dtype),
                                      ctypes.c_void_p(loader.stream_ptr())), "swiglu_fwd")
        ctx.save_for_backward(xc, rs if rs is not None else torch.empty(0, device=x.device))
        ctx.has_scale = rs is not None
        ctx.scale_dtype = None if row_scale is None else row_scale.dtype
        ctx.scale_shape = None if row_scale is None else row_scale.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        L = loader.require_lib()
        x, rs = ctx.saved_tensors
        dy = dy.contiguous()
        f = x.shape[-1] // 2
        rows = x.numel() // (2 * f)
        dx = torch.empty_like(x)
        dscale = torch.zeros(rows, dtype=torch.float32, device=x.device) if ctx.has_scale else None
        loader.check(L.msb_swiglu_bwd(loader.p(dy), loader.p(x), loader.p(dx), loader.p(rs if ctx.has_scale else None),
                                      loader.p(dscale), ctypes.c_longlong(rows), f, code(x.dtype),
                                      ctypes.c_void_p(loader.stream_ptr())), "swiglu_bwd")
        if ctx.has_scale:
            return dx, dscale.to(ctx.scale_dtype).reshape(ctx.scale_shape)
        return dx, None


def swiglu(x, row_scale=None, fused=True):
    if fused and x.is_cuda and loader.use_kernels(x) and x.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(x, row_scale)
    return swiglu_ref(x, row_scale)
