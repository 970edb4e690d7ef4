"""bf16 parameter and fp32 master weight sharing storage ("reuse-fp32-param").

The master weight is kept as the bf16 model parameter plus a 16-bit residual, so the optimizer holds 2 instead of
4 bytes per parameter for it:
    stored = bits(fp32) + 0x8000          (integer add; makes the high half the round-half-up bf16 of the master)
    hi = stored >> 16  -> the bf16 parameter,   lo = stored & 0xffff -> the residual
    bits(fp32) = ((hi << 16) | lo) - 0x8000
(reference: mindspeed/optimizer/optimizer.py:249-280, docs/zh/features/reuse-fp32-param.md:9-13; saves 2 bytes per
parameter, divided by DP with the distributed optimizer.)  The fused kernel ``msb_adam_flat_reuse`` updates such a
pair in place; these helpers are the eager form and the oracle.
"""
from __future__ import annotations

import ctypes
import math

import torch

from ..ops import loader
from ..ops._dtypes import code


def split_fp32(master: torch.Tensor):
    """fp32 -> (bf16 hi, int16 lo)"""
    bits = master.contiguous().view(torch.int32) + 0x8000
    hi = (bits >> 16).to(torch.int16).view(torch.bfloat16)
    lo = (bits & 0xFFFF).to(torch.int32)
    lo = torch.where(lo >= 0x8000, lo - 0x10000, lo).to(torch.int16)
    return hi, lo


def merge_fp32(hi: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    h = hi.contiguous().view(torch.int16).to(torch.int32) << 16
    l = lo.to(torch.int32) & 0xFFFF
    return ((h | l) - 0x8000).view(torch.float32)


def adam_flat_reuse(hi, lo, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, adam_w_mode=True, bias_correction=True,
                    found_inf=None, grad_scale_dev=None):
    """In-place AdamW on a (bf16, residual) master pair."""
    if hi.is_cuda and loader.use_kernels(hi):
        L = loader.require_lib()
        f = ctypes.c_float
        loader.check(L.msb_adam_flat_reuse(loader.p(hi), loader.p(lo), loader.p(g), loader.p(m), loader.p(v),
                                           ctypes.c_longlong(hi.numel()), f(lr), f(beta1), f(beta2), f(eps), f(wd), int(step),
                                           f(grad_scale), int(adam_w_mode), int(bias_correction), loader.p(found_inf),
                                           loader.p(grad_scale_dev), code(g.dtype), ctypes.c_void_p(loader.stream_ptr())),
                     "adam_flat_reuse")
        return
    from ..ops.adam import adam_flat_ref
    p = merge_fp32(hi, lo).clone()
    adam_flat_ref(p, g, m, v, None, lr, beta1, beta2, eps, wd, step, grad_scale, adam_w_mode, bias_correction=bias_correction)
    h2, l2 = split_fp32(p)
    hi.copy_(h2)
    lo.copy_(l2)
