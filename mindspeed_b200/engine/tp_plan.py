"""Tensor-parallel plan for plain ``nn.Linear`` / ``nn.Embedding`` modules of an arbitrary model.

  colwise   weight [out, in] split on out; input replicated (or sequence-sharded and all-gathered with
            sequence_parallel); output is the local slice
  rowwise   weight split on in; input is the local slice; output all-reduced (or reduce-scattered along the
            sequence with sequence_parallel); bias added once after the reduction
  vocab     embedding rows split; out-of-range ids contribute zeros; output all-reduced

The collectives are the autograd-aware mappings of the Megatron-style layers, so backward is handled the same way.
reference: mindspeed/fsdp/distributed/tensor_parallel/* (DTensor plan application in the reference engine).
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel import mappings as M
from ..utils.patterns import match as _match


class ColwiseLinear(nn.Module):
    def __init__(self, lin: nn.Linear, group, sequence_parallel=False):
        super().__init__()
        n, r = M._ws(group), M._rk(group)
        if lin.out_features % n != 0:
            raise ValueError(f"out_features {lin.out_features} not divisible by tensor parallel size {n}")
        per = lin.out_features // n
        self.group, self.sp = group, sequence_parallel
        self.in_features, self.out_features = lin.in_features, per
        self.weight = nn.Parameter(lin.weight.detach()[r * per:(r + 1) * per].clone())
        self.bias = nn.Parameter(lin.bias.detach()[r * per:(r + 1) * per].clone()) if lin.bias is not None else None
        self.weight.tensor_model_parallel = True

    def forward(self, x):
        if self.sp:
            x = M.gather_from_sequence_parallel_region(x, True, self.group)
        else:
            x = M.copy_to_tensor_model_parallel_region(x, self.group)
        return F.linear(x, self.weight, self.bias)


class RowwiseLinear(nn.Module):
    def __init__(self, lin: nn.Linear, group, sequence_parallel=False):
        super().__init__()
        n, r = M._ws(group), M._rk(group)
        if lin.in_features % n != 0:
            raise ValueError(f"in_features {lin.in_features} not divisible by tensor parallel size {n}")
        per = lin.in_features // n
        self.group, self.sp = group, sequence_parallel
        self.in_features, self.out_features = per, lin.out_features
        self.weight = nn.Parameter(lin.weight.detach()[:, r * per:(r + 1) * per].clone())
        self.bias = nn.Parameter(lin.bias.detach().clone()) if lin.bias is not None else None
        self.weight.tensor_model_parallel = True

    def forward(self, x):
        y = F.linear(x, self.weight)
        if self.sp:
            y = M.reduce_scatter_to_sequence_parallel_region(y, self.group)
        else:
            y = M.reduce_from_tensor_model_parallel_region(y, self.group)
        return y if self.bias is None else y + self.bias


class VocabParallelEmbed(nn.Module):
    def __init__(self, emb: nn.Embedding, group):
        super().__init__()
        n, r = M._ws(group), M._rk(group)
        if emb.num_embeddings % n != 0:
            raise ValueError("vocabulary not divisible by tensor parallel size")
        per = emb.num_embeddings // n
        self.group, self.lo, self.hi = group, r * per, (r + 1) * per
        self.weight = nn.Parameter(emb.weight.detach()[self.lo:self.hi].clone())
        self.weight.tensor_model_parallel = True

    def forward(self, ids):
        mask = (ids < self.lo) | (ids >= self.hi)
        local = (ids - self.lo).masked_fill(mask, 0)
        out = F.embedding(local, self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return M.reduce_from_tensor_model_parallel_region(out, self.group)


_STYLES = {"colwise": (nn.Linear, ColwiseLinear), "rowwise": (nn.Linear, RowwiseLinear), "vocab": (nn.Embedding, VocabParallelEmbed)}


def apply_tp_plan(model: nn.Module, rules: Dict[str, str], group, sequence_parallel: bool = False) -> int:
    """Replace every module whose qualified name matches a rule; returns the number of replaced modules."""
    if M._ws(group) == 1:
        return 0
    done = 0
    for name, mod in list(model.named_modules()):
        for pat, style in rules.items():
            if not _match(name, pat):
                continue
            want, cls = _STYLES[style]
            if not isinstance(mod, want):
                raise TypeError(f"tp plan rule {pat!r} ({style}) matched {name!r} of type {type(mod).__name__}")
            new = cls(mod, group) if style == "vocab" else cls(mod, group, sequence_parallel)
            parent = model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], new)
            done += 1
            break
    return done
