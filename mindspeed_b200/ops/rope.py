"""Rotary position embedding on (possibly strided, packed) heads.

``apply_rope(t, cos, sin)`` rotates ``t`` [s, b, n, d] (any strides with contiguous last dim).
``apply_rope_packed_qkv_`` rotates the q and k heads of a packed QKV activation in place.
reference semantics: mindspeed/core/fusions/fused_rope.py:28-74 (mode 0 = rotate-half, mode 1 = interleaved).
"""
from __future__ import annotations

import ctypes

import torch

from . import loader
from ._dtypes import code


def _rotate_half(x, interleaved):
    if not interleaved:
        x1, x2 = x.chunk(2, dim=-1)
        return torch.cat((-x2, x1), dim=-1)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).reshape(x.shape)


def apply_rope_ref(t, cos, sin, interleaved=False):
    """t [s,b,n,d]; cos/sin [s, rot_dim] fp32."""
    rot = cos.shape[-1]
    tr, tp = t[..., :rot].float(), t[..., rot:]
    c, s = cos.reshape(cos.shape[0], 1, 1, rot), sin.reshape(sin.shape[0], 1, 1, rot)
    out = tr * c + _rotate_half(tr, interleaved) * s
    return torch.cat((out.to(t.dtype), tp), dim=-1)


def _launch(x, y, cos, sin, tokens, heads, head_dim, ts_in, hs_in, ts_out, hs_out, tokens_per_pos, group_heads, rope_heads,
            interleaved, backward):
    L = loader.require_lib()
    loader.check(L.msb_rope(loader.p(x), loader.p(y), loader.p(cos), loader.p(sin), ctypes.c_longlong(tokens), heads,
                            head_dim, cos.shape[-1], ctypes.c_longlong(ts_in), ctypes.c_longlong(hs_in),
                            ctypes.c_longlong(ts_out), ctypes.c_longlong(hs_out), tokens_per_pos, group_heads, rope_heads,
                            int(interleaved), int(backward), code(x.dtype), ctypes.c_void_p(loader.stream_ptr())), "rope")


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, cos, sin, interleaved):
        s, b, n, d = t.shape
        tc = t if (t.stride(-1) == 1 and t.stride(0) == b * t.stride(1)) else t.contiguous()
        y = torch.empty((s, b, n, d), dtype=t.dtype, device=t.device)
        _launch(tc, y, cos, sin, s * b, n, d, tc.stride(1), tc.stride(2), n * d, d, b, 1, 1, interleaved, False)
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = interleaved
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        dy = dy.contiguous()
        s, b, n, d = dy.shape
        dx = torch.empty_like(dy)
        _launch(dy, dx, cos, sin, s * b, n, d, n * d, d, n * d, d, b, 1, 1, ctx.interleaved, True)
        return dx, None, None, None


def apply_rope(t, cos, sin, interleaved=False, fused=True):
    if fused and t.is_cuda and loader.use_kernels(t):
        return _RopeFn.apply(t, cos.float().contiguous(), sin.float().contiguous(), interleaved)
    return apply_rope_ref(t, cos, sin, interleaved)


def rope_packed_qkv_(qkv, cos, sin, num_groups, q_per_group, head_dim, interleaved=False, backward=False):
    """In place on ``qkv`` [s, b, groups*(q_per_group+2)*head_dim]: rotate q and k heads, leave v."""
    s, b, w = qkv.shape
    gh = q_per_group + 2
    assert w == num_groups * gh * head_dim and qkv.is_contiguous()
    if qkv.is_cuda and loader.use_kernels(qkv):
        _launch(qkv, qkv, cos, sin, s * b, num_groups * gh, head_dim, w, head_dim, w, head_dim, b, gh, q_per_group + 1,
                interleaved, backward)
        return qkv
    v = qkv.view(s, b, num_groups, gh, head_dim)
    sgn = -1.0 if backward else 1.0
    part = v[:, :, :, :q_per_group + 1].reshape(s, b, num_groups * (q_per_group + 1), head_dim)
    out = apply_rope_ref(part, cos, sin * sgn, interleaved)
    v[:, :, :, :q_per_group + 1] = out.view(s, b, num_groups, q_per_group + 1, head_dim)
    return qkv
