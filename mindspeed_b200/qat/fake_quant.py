"""Fake-quantised linears for quantisation-aware training.

``fake_quantize(x, bits, group, symmetric)`` rounds to a ``bits``-bit integer grid per group of ``group`` consecutive
elements of the last dimension (group = -1: per row) and returns the de-quantised value; the backward is the
straight-through estimator with the clipped range masked out.  Schemes: W4A16, W8A16 (weights only), W4A4, W8A8
(weights + activations; activations per token).
reference: mindspeed/core/qat/* (fake-quant linear variants W4A16 / W8A16 / W4A4).
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils.patterns import match as _match


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bits, group, symmetric):
        shp = x.shape
        g = shp[-1] if group in (-1, None) or group >= shp[-1] else group
        if shp[-1] % g != 0:
            raise ValueError(f"last dimension {shp[-1]} not divisible by the quantisation group {g}")
        xf = x.float().reshape(-1, g)
        if symmetric:
            qmax = 2 ** (bits - 1) - 1
            scale = xf.abs().amax(dim=1, keepdim=True).clamp_min(1e-12) / qmax
            q = torch.round(xf / scale).clamp(-qmax - 1, qmax)
            out = q * scale
            mask = (xf / scale).abs() <= qmax + 1
        else:
            qmax = 2 ** bits - 1
            lo, hi = xf.amin(dim=1, keepdim=True), xf.amax(dim=1, keepdim=True)
            scale = (hi - lo).clamp_min(1e-12) / qmax
            zp = torch.round(-lo / scale)
            q = (torch.round(xf / scale) + zp).clamp(0, qmax)
            out = (q - zp) * scale
            mask = torch.ones_like(xf, dtype=torch.bool)
        ctx.save_for_backward(mask.reshape(shp))
        return out.reshape(shp).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return g * mask.to(g.dtype), None, None, None


def fake_quantize(x, bits: int = 8, group: int = -1, symmetric: bool = True):
    return _FakeQuantSTE.apply(x, bits, group, symmetric)


@dataclasses.dataclass
class QATConfig:
    scheme: str = "W4A16"                 # W4A16 | W8A16 | W4A4 | W8A8
    weight_group: int = 128
    symmetric: bool = True
    modules: Sequence[str] = ("**",)      # name patterns of nn.Linear modules to convert
    skip: Sequence[str] = ("**.output_layer", "**lm_head", "**.router", "**.gate")

    def bits(self):
        s = self.scheme.upper()
        if not (s.startswith("W") and "A" in s):
            raise ValueError(f"bad QAT scheme {self.scheme}")
        wb, ab = s[1:].split("A")
        return int(wb), int(ab)


class FakeQuantLinear(nn.Module):
    """Wraps the weight (and optionally the input) of a linear map in fake quantisation; parameters stay full precision."""

    def __init__(self, weight: nn.Parameter, bias: Optional[nn.Parameter], cfg: QATConfig):
        super().__init__()
        self.weight, self.bias, self.cfg = weight, bias, cfg
        self.w_bits, self.a_bits = cfg.bits()

    def quantized_weight(self):
        return fake_quantize(self.weight, self.w_bits, self.cfg.weight_group, self.cfg.symmetric)

    def forward(self, x):
        if self.a_bits < 16:
            x = fake_quantize(x, self.a_bits, -1, self.cfg.symmetric)      # per token
        return F.linear(x, self.quantized_weight(), self.bias)


def apply_qat(model: nn.Module, cfg: QATConfig) -> int:
    """Replace matching ``nn.Linear`` modules; tensor-parallel linears of this framework get their weight hooked
    instead (their forward reads ``self.weight`` through a property-like pre-forward swap)."""
    n = 0
    for name, mod in list(model.named_modules()):
        if not name or not any(_match(name, p) for p in cfg.modules) or any(_match(name, p) for p in cfg.skip):
            continue
        if type(mod) is nn.Linear:
            parent = model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], FakeQuantLinear(mod.weight, mod.bias, cfg))
            n += 1
        elif type(mod).__name__ in ("ColumnParallelLinear", "RowParallelLinear", "TEColumnParallelLinear", "TERowParallelLinear"):
            _hook_parallel_linear(mod, cfg)
            n += 1
    return n


def _hook_parallel_linear(mod, cfg: QATConfig):
    wb, ab = cfg.bits()
    orig_forward = mod.forward

    def forward(input_, *a, **kw):
        if ab < 16:
            input_ = fake_quantize(input_, ab, -1, cfg.symmetric)
        real = mod.weight
        # run the layer's own forward (communication included) on the fake-quantised weight
        qw = fake_quantize(real, wb, cfg.weight_group, cfg.symmetric)
        if "weight" in orig_forward.__code__.co_varnames:
            return orig_forward(input_, qw, *a[1:], **kw) if a else orig_forward(input_, weight=qw, **kw)
        object.__setattr__(mod, "_qat_real_weight", real)
        try:
            mod._parameters.pop("weight")
            object.__setattr__(mod, "weight", qw)
            return orig_forward(input_, *a, **kw)
        finally:
            object.__delattr__(mod, "weight")
            mod._parameters["weight"] = real
    mod.forward = forward
