"""Fused feed-forward op with the call shape of the reference's inference-style FFN, and quantised grouped GEMMs.

``ffn(x, weight1, weight2, activation, expert_tokens=None, bias1=None, bias2=None)``
    y = act(x @ weight1 + bias1) @ weight2 + bias2, dense (weights [K, N]) or per expert (weights [E, K, N] with
    ``expert_tokens`` rows per expert; x sorted by expert).  GEMMs run on the tcgen05 kernels (dense: ``ops.gemm``, experts: the
    one-launch grouped kernel), gated activations (``swiglu`` / ``geglu`` / ``reglu``) on the fused activation kernel.
    reference: mindspeed/ops/ffn.py:29-68 over mindspeed/ops/csrc/cann/ffn.cpp (aclnnFFNV3).

``weight_quant_grouped_gemm(x, qweight, scale, offset, tokens_per_expert)``
    int8 (or int4-in-int8) weights with per-output-channel scale / offset: w = (q + offset) * scale, dequantised per expert on
    the way into the grouped GEMM.  reference: mindspeed/ops/csrc/cann/weight_quant_gmm.cpp (npu_weight_quant_gmm).

``quant_grouped_gemm(qx, qweight, scale, per_token_scale, tokens_per_expert, out_dtype)``
    int8 activations x int8 weights accumulated in int32, then scaled per output channel and per token.
    reference: mindspeed/ops/csrc/cann/quant_gmm.cpp (npu_quant_gmm).
"""
from __future__ import annotations

from typing import Optional, Sequence, Union

import torch
import torch.nn.functional as F

from .activation import swiglu
from .grouped_gemm import grouped_gemm

_GATED = {"swiglu": F.silu, "geglu": F.gelu, "reglu": F.relu}
_PLAIN = {"gelu": F.gelu, "relu": F.relu, "silu": F.silu, "fastgelu": lambda t: F.gelu(t, approximate="tanh")}


def _act(h: torch.Tensor, activation: str) -> torch.Tensor:
    name = activation.lower()
    if name == "swiglu":
        return swiglu(h, fused=h.is_cuda)
    if name in _GATED:
        g, u = h.chunk(2, dim=-1)
        return _GATED[name](g) * u
    if name in _PLAIN:
        return _PLAIN[name](h)
    raise ValueError(f"unknown activation {activation!r}: one of {sorted(_GATED) + sorted(_PLAIN)}")


def ffn(x: torch.Tensor, weight1: torch.Tensor, weight2: torch.Tensor, activation: str = "gelu",
        expert_tokens: Optional[Union[torch.Tensor, Sequence[int]]] = None, bias1: Optional[torch.Tensor] = None,
        bias2: Optional[torch.Tensor] = None) -> torch.Tensor:
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if expert_tokens is None:
        if weight1.dim() != 2:
            raise ValueError("dense ffn takes [K, N] weights; pass expert_tokens for stacked expert weights")
        h = x2 @ weight1 if not x2.is_cuda else _dense(x2, weight1)
        if bias1 is not None:
            h = h + bias1
        a = _act(h, activation)
        y = a @ weight2 if not a.is_cuda else _dense(a, weight2)
        if bias2 is not None:
            y = y + bias2
        return y.reshape(*lead, y.shape[-1])
    if weight1.dim() != 3:
        raise ValueError("expert ffn takes stacked [E, K, N] weights")
    counts = expert_tokens
    h = grouped_gemm(x2, weight1, counts)
    if bias1 is not None:
        h = h + _expand_bias(bias1, counts, h)
    a = _act(h, activation)
    y = grouped_gemm(a, weight2, counts)
    if bias2 is not None:
        y = y + _expand_bias(bias2, counts, y)
    return y.reshape(*lead, y.shape[-1])


def _dense(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x2 [M, K] @ w [K, N] on the own GEMM when the shapes allow it (the kernel takes the weight as [N, K])."""
    from . import gemm as G
    from . import loader
    if x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and loader.lib() is not None and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        return G.linear_dgrad(x2.contiguous(), w.contiguous())        # dy [M, K] @ w [K, N]: the "dgrad" operand layout
    return x2 @ w


def _expand_bias(bias: torch.Tensor, counts, like: torch.Tensor) -> torch.Tensor:
    c = counts if torch.is_tensor(counts) else torch.tensor(list(counts))
    return torch.repeat_interleave(bias.to(like.dtype), c.to(bias.device), dim=0, output_size=like.shape[0])


def weight_quant_grouped_gemm(x: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor, offset: Optional[torch.Tensor],
                              tokens_per_expert) -> torch.Tensor:
    """qweight [E, K, N] int8; scale / offset [E, N] (per output channel).  Returns x's dtype."""
    w = qweight.to(torch.float32)
    if offset is not None:
        w = w + offset.to(torch.float32).unsqueeze(1)
    w = (w * scale.to(torch.float32).unsqueeze(1)).to(x.dtype)
    return grouped_gemm(x, w, tokens_per_expert)


def quant_grouped_gemm(qx: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor, per_token_scale: Optional[torch.Tensor],
                       tokens_per_expert, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """qx [M, K] int8, qweight [E, K, N] int8, scale [E, N], per_token_scale [M] or None."""
    counts = tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)
    out = torch.empty(qx.shape[0], qweight.shape[2], dtype=torch.float32, device=qx.device)
    row = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        a, b = qx[row:row + n], qweight[e]
        if qx.is_cuda and n > 16 and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
            acc = torch._int_mm(a.contiguous(), b.contiguous()).to(torch.float32)      # int8 tensor cores, int32 accumulate
        else:
            acc = (a.to(torch.int32) @ b.to(torch.int32)).to(torch.float32) if not qx.is_cuda else a.float() @ b.float()
        out[row:row + n] = acc * scale[e].to(torch.float32)
        row += n
    if per_token_scale is not None:
        out = out * per_token_scale.to(torch.float32).unsqueeze(1)
    return out.to(out_dtype)
