"""Row gather / weighted scatter-add for MoE token permutation (csrc/kernels/permute.cu)."""
from __future__ import annotations

import ctypes

import torch

from . import loader
from ._dtypes import code


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx):
        L = loader.require_lib()
        x = x.contiguous()
        idx = idx.contiguous().long()
        out = torch.empty(idx.numel(), x.shape[1], dtype=x.dtype, device=x.device)
        loader.check(L.msb_gather_rows(loader.p(x), loader.p(idx), loader.p(out), ctypes.c_longlong(idx.numel()), x.shape[1],
                                       code(x.dtype), ctypes.c_void_p(loader.stream_ptr())), "gather_rows")
        ctx.save_for_backward(idx)
        ctx.rows = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        return _scatter(g.contiguous(), idx, ctx.rows, None), None


def _scatter(src, idx, rows, weight):
    L = loader.require_lib()
    out = torch.zeros(rows, src.shape[1], dtype=torch.float32, device=src.device)
    loader.check(L.msb_scatter_add_rows(loader.p(src), loader.p(idx), loader.p(weight), loader.p(out),
                                        ctypes.c_longlong(idx.numel()), src.shape[1], code(src.dtype),
                                        ctypes.c_void_p(loader.stream_ptr())), "scatter_add_rows")
    return out.to(src.dtype)


class _ScatterAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, idx, rows, weight):
        idx = idx.contiguous().long()
        src = src.contiguous()
        w = None if weight is None else weight.float().contiguous()
        ctx.save_for_backward(src, idx, w if w is not None else torch.empty(0, device=src.device))
        ctx.has_w = w is not None
        ctx.wdtype = None if weight is None else weight.dtype
        return _scatter(src, idx, rows, w)

    @staticmethod
    def backward(ctx, g):
        src, idx, w = ctx.saved_tensors
        g = g.contiguous()
        gs = _Gather.apply(g, idx)
        dw = None
        if ctx.has_w:
            dw = (gs.float() * src.float()).sum(-1).to(ctx.wdtype)
            gs = gs * w.unsqueeze(-1).to(gs.dtype)
        return gs, None, None, dw


def gather_rows(x, idx):
    return _Gather.apply(x, idx)


def scatter_add_rows(src, idx, rows, weight=None):
    return _ScatterAdd.apply(src, idx, rows, weight)
