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
    d = q.shape[-1]
    return q.dtype == torch.bfloat16 and d == 128 and v.shape[-1] == 128 and q.shape[0] % 128 == 0 and k.shape[0] % 128 == 0


def flash_attention(q, k, v, causal, softmax_scale, return_lse):
    from .flash_sm100_impl import flash_attention as impl
    return impl(q, k, v, causal, softmax_scale, return_lse)
