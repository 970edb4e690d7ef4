"""Python front end of the hand-written sm_100a flash attention (csrc/kernels/flash_attn_sm100.cu)."""
from __future__ import annotations

import ctypes
import math

import torch

from . import loader
from ._dtypes import code


def supports(q, k, v, causal) -> bool:
    L = loader.lib()
    if L is None or not hasattr(L, "msb_flash_fwd"):
        return False
    if not hasattr(L, "msb_flash_fwd2") or not hasattr(L, "msb_flash_bwd"):
        return False
    d = q.shape[-1]
    if not (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and d == 128 and k.shape[-1] == 128 and v.shape[-1] == 128):
        return False
    if causal and k.shape[0] < q.shape[0]:
        return False
    for t in (q, k, v):           # TMA needs a contiguous head dim, 16-byte aligned strides and base
        if t.stride(-1) != 1 or any((st * 2) % 16 for st in t.stride()[:-1]) or t.data_ptr() % 16:
            return False
    return True


def flash_attention(q, k, v, causal, softmax_scale, return_lse):
    from .flash_sm100_impl import flash_attention as impl
    return impl(q, k, v, causal, softmax_scale, return_lse)
