"""Module converters of the engine's quantisation plan: ``nn.Linear`` -> a linear whose three GEMMs run on fp8 operands.

``convert_linears(model, QuantizeConfig)`` replaces the linears selected by the plan's patterns with
``models.te_compat.Fp8Linear`` under the plan's recipe; parameters are shared with the original module, so tensor-parallel
styles, expert sharding and full sharding applied afterwards see the same tensors.  ``MXFP8Linear`` / ``MXFP8GroupedLinear``
are the stand-alone modules of the micro-scaling recipe (a grouped linear = one weight per expert, rows of the input split by
``tokens_per_expert``); on a GPU without a block-scaled kernel for the recipe they compute on the dequantised operands, which
is the arithmetic the block-scaled tensor-core instruction defines.
reference: mindspeed/fsdp/quantization/{converter/model_converter.py,converter/mx_converter.py,module/linear_mxfp8.py,
module/gmm_mxfp8.py}.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn

from ..models.te_compat import Fp8Linear, MXFP8Scaling, _FakeQuantLinearFn
from ..utils.patterns import match as _match


def selected(name: str, apply: List[str], ignored: List[str]) -> bool:
    if any(_match(name, p) for p in ignored):
        return False
    return not apply or any(_match(name, p) for p in apply)


def convert_linears(model: nn.Module, plan) -> int:
    rec = plan.recipe()
    n = 0
    for name, mod in list(model.named_modules()):
        if type(mod) is not nn.Linear or not selected(name, plan.apply_modules, plan.ignored_modules):
            continue
        parent = model
        parts = name.split(".")
        for p in parts[:-1]:
            parent = getattr(parent, p)
        setattr(parent, parts[-1], Fp8Linear(mod, rec))
        n += 1
    return n


class MXFP8Linear(nn.Linear):
    """``nn.Linear`` computing y = x W^T with both operands in micro-scaled fp8 (and both gradients likewise)."""

    def __init__(self, in_features, out_features, bias=True, fp8_format="hybrid", device=None, dtype=None):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.recipe = MXFP8Scaling(fp8_format=fp8_format)

    def forward(self, x):
        y = _FakeQuantLinearFn.apply(x, self.weight, self.recipe, None)
        return y if self.bias is None else y + self.bias


class MXFP8GroupedLinear(nn.Module):
    """E weights [E, out, in]; rows of ``x`` are grouped by expert (``tokens_per_expert`` rows each, in order)."""

    def __init__(self, num_experts, in_features, out_features, fp8_format="hybrid", device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features, device=device, dtype=dtype))
        for e in range(num_experts):
            nn.init.kaiming_uniform_(self.weight[e], a=5 ** 0.5)
        self.recipe = MXFP8Scaling(fp8_format=fp8_format)

    def forward(self, x, tokens_per_expert):
        counts = [int(c) for c in tokens_per_expert]
        if sum(counts) != x.shape[0]:
            raise ValueError(f"tokens_per_expert sums to {sum(counts)}, input has {x.shape[0]} rows")
        outs, at = [], 0
        for e, c in enumerate(counts):
            if c:
                outs.append(_FakeQuantLinearFn.apply(x[at:at + c], self.weight[e], self.recipe, None))
            at += c
        if not outs:
            return x.new_zeros(0, self.weight.shape[1]) + 0.0 * self.weight.sum()
        return torch.cat(outs, dim=0)
