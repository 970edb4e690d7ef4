"""Fused AdamW / gradient-norm kernels on flat fp32 shards (csrc/kernels/adam.cu)."""
from __future__ import annotations

import ctypes
import math

import torch

from . import loader
from ._dtypes import code


def adam_flat_ref(p, g, m, v, p16, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, adam_w_mode=True, ema=None,
                  ema_decay=0.0, bias_correction=True, maximize=False):
    gf = g.float() * grad_scale
    if maximize:
        gf = -gf
    if not adam_w_mode:
        gf = gf + wd * p
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step if bias_correction else 1.0
    bc2 = 1 - beta2 ** step if bias_correction else 1.0
    denom = v.sqrt() / math.sqrt(bc2) + eps
    if adam_w_mode:
        p.mul_(1 - lr * wd)
    p.addcdiv_(m / bc1, denom, value=-lr)
    if p16 is not None:
        p16.copy_(p)
    if ema is not None:
        ema.mul_(ema_decay).add_(p, alpha=1 - ema_decay)


def adam_flat(p, g, m, v, p16, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, adam_w_mode=True, ema=None,
              ema_decay=0.0, bias_correction=True, maximize=False, found_inf=None, grad_scale_dev=None):
    """In-place AdamW step on flat fp32 ``p, m, v`` from ``g``; writes the low-precision copy ``p16``."""
    if not (p.is_cuda and loader.use_kernels(p)):
        return adam_flat_ref(p, g, m, v, p16, lr, beta1, beta2, eps, wd, step, grad_scale, adam_w_mode, ema, ema_decay,
                             bias_correction, maximize)
    L = loader.require_lib()
    assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
    f = ctypes.c_float
    loader.check(L.msb_adam_flat(loader.p(p), loader.p(g), loader.p(m), loader.p(v), loader.p(p16), loader.p(ema),
                                 ctypes.c_longlong(p.numel()), f(lr), f(beta1), f(beta2), f(eps), f(wd), int(step),
                                 f(grad_scale), f(ema_decay), int(adam_w_mode), int(maximize), int(bias_correction),
                                 loader.p(found_inf), loader.p(grad_scale_dev), code(g.dtype),
                                 code(p16.dtype) if p16 is not None else 1, ctypes.c_void_p(loader.stream_ptr())),
                 "adam_flat")


_norm_scratch = {}


def l2norm_sq(g, out=None, accumulate=False):
    """Sum of squares of ``g`` as a 1-element fp32 device tensor (no host sync)."""
    if not (g.is_cuda and loader.use_kernels(g)):
        r = g.float().pow(2).sum().reshape(1)
        if out is not None:
            out.copy_(out + r if accumulate else r)
            return out
        return r
    L = loader.require_lib()
    n = L.msb_l2norm_sq_scratch_elems()
    sc = _norm_scratch.get(g.device)
    if sc is None:
        sc = torch.empty(n, dtype=torch.float32, device=g.device)
        _norm_scratch[g.device] = sc
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=g.device)
    loader.check(L.msb_l2norm_sq(loader.p(g.contiguous()), ctypes.c_longlong(g.numel()), loader.p(sc), loader.p(out),
                                 int(accumulate), code(g.dtype), ctypes.c_void_p(loader.stream_ptr())), "l2norm_sq")
    return out


def clip_coef(norm_sq, max_norm, coef, found_inf=None, norm_out=None):
    L = loader.require_lib()
    loader.check(L.msb_clip_coef(loader.p(norm_sq), ctypes.c_float(max_norm), loader.p(coef), loader.p(found_inf),
                                 loader.p(norm_out), ctypes.c_void_p(loader.stream_ptr())), "clip_coef")


def scale_(x, scale=1.0, scale_dev=None):
    if not (x.is_cuda and loader.use_kernels(x)):
        x.mul_(scale if scale_dev is None else scale * scale_dev.item())
        return x
    L = loader.require_lib()
    loader.check(L.msb_scale(loader.p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(scale), loader.p(scale_dev),
                             code(x.dtype), ctypes.c_void_p(loader.stream_ptr())), "scale")
    return x
