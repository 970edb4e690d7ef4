"""Transformer-Engine-compatible modules and fp8 recipes.

Modules (same constructor / forward contract as the Megatron ``TE*`` spec classes, so layer specs written for them
run unchanged):

  TEColumnParallelLinear, TERowParallelLinear     tensor-parallel linears with pluggable communication back ends
                                                  (library / chunked / fused) and optional fp8 compute
  TELayerNormColumnParallelLinear                 norm fused in front of a column-parallel linear
  TEGroupedLinear                                 per-expert weights, grouped GEMM (bf16 or block-scaled fp8)
  TEDotProductAttention                           core attention with the context-parallel strategy selected by config
  TENorm                                          LayerNorm / RMSNorm factory

fp8:  ``with fp8_autocast(enabled=True, fp8_recipe=BlockwiseScaling()):`` switches the linears above to fp8 compute.

  recipe        scaling granularity                              compute path
  delayed       per tensor, scale from an amax history           fp8 round trip of operands + bf16 GEMM
  tensorwise    per tensor, scale from the current amax          fp8 round trip of operands + bf16 GEMM
  blockwise     activations 1x128, weights 128x128               block-scaled tcgen05 fp8 GEMM (ops/gemm_fp8.py)
  mxfp8         1x32 blocks, power-of-two (e8m0) scales          fp8 round trip of operands + bf16 GEMM
  formats: E4M3 (max 448) forward / E5M2 (max 57344) for gradients in "hybrid".

The quantised weight (and its transpose) is cached per module across micro-batches and dropped by
``clear_fp8_weight_cache()`` after the optimizer step.
reference: mindspeed/te/pytorch/module/linear.py:31-641, layernorm_column_parallel_linear.py:61-287,
grouped_linear.py:47-412, fp8/recipes/*.py, fp8/constants.py:14-90, fp8/reuse.py:106-266, fp8/fp8.py:12-93.
"""
from __future__ import annotations

import contextlib
import dataclasses
import weakref
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import quant as Q
from ..ops.gemm_fp8 import fp8_blockwise_linear, fp8_grouped_gemm
from ..ops.grouped_gemm import grouped_gemm
from ..parallel import mappings as M
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .norms import build_norm

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
FORMATS = {"e4m3": (E4M3, E4M3), "hybrid": (E4M3, E5M2)}


# ---- recipes ---------------------------------------------------------------------------------------------------
@dataclasses.dataclass
class Recipe:
    fp8_format: str = "hybrid"
    name = "base"

    def dtype_for(self, key: str):
        fwd, bwd = FORMATS[self.fp8_format]
        return bwd if key == "grads" else fwd

    def round_trip(self, t: torch.Tensor, key: str, state: Optional[dict] = None) -> torch.Tensor:
        """Quantise ``t`` for role ``key`` ("inputs" | "weight" | "grads") and return its dequantised value."""
        raise NotImplementedError


@dataclasses.dataclass
class TensorwiseScaling(Recipe):
    name = "tensorwise"

    def round_trip(self, t, key, state=None):
        dt = self.dtype_for(key)
        fmax = Q._fmax(dt)
        scale = t.detach().abs().amax().float().clamp_min(1e-30) / fmax
        return ((t.float() / scale).clamp(-fmax, fmax).to(dt).float() * scale).to(t.dtype)


@dataclasses.dataclass
class DelayedScaling(Recipe):
    """Scale from the maximum (or most recent) of the last ``amax_history_len`` amax values; the current tensor's
    amax only enters the history, so quantisation needs no reduction before the cast."""
    amax_history_len: int = 16
    amax_compute_algo: str = "max"
    margin: int = 0
    name = "delayed"

    def round_trip(self, t, key, state=None):
        dt = self.dtype_for(key)
        fmax = Q._fmax(dt)
        hist: List[float] = state.setdefault(key, []) if state is not None else []
        cur = float(t.detach().abs().amax())
        if hist:
            amax = max(hist) if self.amax_compute_algo == "max" else hist[-1]
        else:
            amax = cur
        hist.append(cur)
        if len(hist) > self.amax_history_len:
            del hist[0]
        scale = max(amax, 1e-30) / fmax * (2.0 ** self.margin)
        return ((t.float() / scale).clamp(-fmax, fmax).to(dt).float() * scale).to(t.dtype)


@dataclasses.dataclass
class BlockwiseScaling(Recipe):
    name = "blockwise"

    def round_trip(self, t, key, state=None):
        t2 = t.reshape(-1, t.shape[-1])
        dt = self.dtype_for(key)
        if key == "weight" and t2.shape[0] % 128 == 0 and t2.shape[1] % 128 == 0:
            q, s = Q.quant_128x128(t2, dtype=dt)
            out = (q.float().view(t2.shape[0] // 128, 128, t2.shape[1] // 128, 128) * s[:, None, :, None]).view(t2.shape)
        else:
            q, s = Q.quant_1x128(t2, dtype=dt)
            out = (q.float().view(t2.shape[0], -1, 128) * s.unsqueeze(-1)).view(t2.shape)
        return out.view(t.shape).to(t.dtype)


@dataclasses.dataclass
class MXFP8Scaling(Recipe):
    """Micro-scaling fp8: blocks of 32 elements ALONG THE CONTRACTION AXIS of the GEMM that consumes the tensor share one
    power-of-two (e8m0) scale.  The three GEMMs of a linear contract over different axes - forward over the input features,
    the data gradient over the output features, the weight gradient over the tokens - so every operand is quantised twice,
    once per axis it is contracted over (``axis_aware``; reference: the dual-axis quantisation of
    mindspeed/te/pytorch/fp8/recipes/mxfp8_scaling_recipe.py:68-132).  An axis whose length is not a multiple of 32 is
    zero-padded for the quantisation."""
    name = "mxfp8"
    axis_aware = True

    def round_trip(self, t, key, state=None, axis: int = -1):
        n = t.shape[axis]
        pad = -n % 32
        if pad:
            t2 = torch.nn.functional.pad(t.movedim(axis, -1), (0, pad))
            q, e = Q.quant_mx(t2, axis=-1, dtype=self.dtype_for(key))
            return Q.dequant_mx(q, e, axis=-1)[..., :n].movedim(-1, axis).to(t.dtype)
        q, e = Q.quant_mx(t, axis=axis, dtype=self.dtype_for(key))
        return Q.dequant_mx(q, e, axis=axis).to(t.dtype)


RECIPES = {"delayed": DelayedScaling, "tensorwise": TensorwiseScaling, "blockwise": BlockwiseScaling, "mxfp8": MXFP8Scaling,
           "mxfp8-32x32": MXFP8Scaling}


def recipe_from_args(args) -> Optional[Recipe]:
    fmt = getattr(args, "fp8_format", None) or getattr(args, "fp8", None)
    if not fmt:
        return None
    cls = RECIPES[getattr(args, "fp8_recipe", "delayed")]
    kw = {}
    if cls is DelayedScaling:                       # --fp8-amax-history-len / --fp8-amax-compute-algo / --fp8-margin
        kw = dict(amax_history_len=int(getattr(args, "fp8_amax_history_len", 16) or 16),
                  amax_compute_algo=getattr(args, "fp8_amax_compute_algo", "max") or "max", margin=int(getattr(args, "fp8_margin", 0) or 0))
    return cls(fp8_format="hybrid" if fmt == "hybrid" else "e4m3", **kw)


# ---- global fp8 state ------------------------------------------------------------------------------------------
class _FP8State:
    enabled = False
    recipe: Optional[Recipe] = None
    modules: "weakref.WeakSet" = weakref.WeakSet()


@contextlib.contextmanager
def fp8_autocast(enabled: bool = True, fp8_recipe: Optional[Recipe] = None, fp8_group=None):
    prev = (_FP8State.enabled, _FP8State.recipe)
    _FP8State.enabled, _FP8State.recipe = enabled, (fp8_recipe or DelayedScaling()) if enabled else None
    try:
        yield
    finally:
        _FP8State.enabled, _FP8State.recipe = prev


def fp8_enabled() -> bool:
    return _FP8State.enabled


def clear_fp8_weight_cache():
    """Call after the optimizer step: cached quantised weights are stale once the weights moved."""
    for m in list(_FP8State.modules):
        m._fp8_wcache.clear()


class _FakeQuantLinearFn(torch.autograd.Function):
    """y = rt(x) @ rt(w)^T ; dx = rt(dy) @ rt(w) ; dw = rt(dy)^T @ rt(x)  (rt = fp8 round trip, straight-through)."""

    @staticmethod
    def forward(ctx, x, w, recipe, state):
        xq = recipe.round_trip(x, "inputs", state)
        wq = recipe.round_trip(w, "weight", state)
        ctx.recipe, ctx.state = recipe, state
        if getattr(recipe, "axis_aware", False):
            ctx.save_for_backward(x, w)                 # backward re-quantises along the axes its GEMMs contract over
        else:
            ctx.save_for_backward(xq, wq)
        return torch.matmul(xq, wq.t())

    @staticmethod
    def backward(ctx, dy):
        r, st = ctx.recipe, ctx.state
        if getattr(r, "axis_aware", False):
            x, w = ctx.saved_tensors
            dx = dw = None
            if ctx.needs_input_grad[0]:                 # dx = dy @ w: contraction over the output features
                dx = torch.matmul(r.round_trip(dy, "grads", st, axis=-1), r.round_trip(w, "weight", st, axis=0))
            if ctx.needs_input_grad[1]:                 # dw = dy^T @ x: contraction over the tokens
                d2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
                dw = torch.matmul(r.round_trip(d2, "grads", st, axis=0).t(), r.round_trip(x2, "inputs", st, axis=0))
            return dx, dw, None, None
        xq, wq = ctx.saved_tensors
        dq = r.round_trip(dy, "grads", st)
        dx = torch.matmul(dq, wq) if ctx.needs_input_grad[0] else None
        dw = torch.matmul(dq.reshape(-1, dq.shape[-1]).t(), xq.reshape(-1, xq.shape[-1])) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


class OnlineComparison:
    """``--te-comparison-with-bf16`` / ``--te-comparison-with-cpu``: every low-precision linear is also computed in the
    unquantised working precision on the device, or in fp32 on the host, and the relative error of the fp8 result
    (``|y_fp8 - y_ref|_F / |y_ref|_F``) is recorded; an error above ``limit`` stops the run with the offending layer's shape.
    reference: the online comparison of the reference's low-precision modules (``--te-comparison-with-cpu/-bf16``,
    mindspeed/features_manager/megatron_basic/transformer_engine_basic.py)."""
    mode: Optional[str] = None           # None | "bf16" | "cpu"
    limit: float = 0.25
    records: List[dict] = []

    @classmethod
    def configure(cls, with_bf16: bool = False, with_cpu: bool = False, limit: float = 0.25):
        cls.mode = "cpu" if with_cpu else ("bf16" if with_bf16 else None)
        cls.limit, cls.records = limit, []

    @classmethod
    def check(cls, x, w, y):
        with torch.no_grad():
            if cls.mode == "cpu":
                ref = torch.matmul(x.detach().float().cpu(), w.detach().float().cpu().t())
                got = y.detach().float().cpu()
            else:
                ref = torch.matmul(x.detach(), w.detach().t()).float()
                got = y.detach().float()
            err = float((got - ref).norm() / ref.norm().clamp_min(1e-30))
        rec = {"shape": (tuple(x.shape), tuple(w.shape)), "reference": cls.mode, "rel_err": err}
        cls.records.append(rec)
        if len(cls.records) > 4096:
            del cls.records[:2048]
        if not (err <= cls.limit):
            raise RuntimeError(f"low-precision linear x{tuple(x.shape)} @ w{tuple(w.shape)}^T deviates from the {cls.mode} "
                               f"reference by {err:.4f} (limit {cls.limit})")


def fp8_linear(x, w, module=None, recipe: Optional[Recipe] = None):
    """Local (un-sharded) fp8 linear under ``recipe`` (default: the active autocast recipe)."""
    recipe = recipe or _FP8State.recipe
    state = module._fp8_state if module is not None else None
    if isinstance(recipe, BlockwiseScaling) and x.shape[-1] % 128 == 0 and w.shape[0] % 128 == 0:
        cache = module._fp8_wcache if module is not None else None
        y = fp8_blockwise_linear(x, w, cache, recipe.dtype_for("grads"))
    else:
        y = _FakeQuantLinearFn.apply(x, w, recipe, state)
    if OnlineComparison.mode is not None:
        OnlineComparison.check(x, w, y)
    return y


class _Fp8Mixin:
    def _init_fp8(self):
        self._fp8_state: Dict[str, list] = {}
        self._fp8_wcache: Dict[str, torch.Tensor] = {}
        _FP8State.modules.add(self)


# ---- modules ---------------------------------------------------------------------------------------------------
class TEColumnParallelLinear(ColumnParallelLinear, _Fp8Mixin):
    def __init__(self, input_size, output_size, *, config, init_method, gather_output=False, bias=True, skip_bias_add=False,
                 is_expert=False, skip_weight_param_allocation=False, tp_comm_buffer_name=None, tp_group=None, stride=1, **_):
        super().__init__(input_size, output_size, config=config, init_method=init_method, bias=bias, gather_output=gather_output,
                         skip_bias_add=skip_bias_add, is_expert=is_expert, skip_weight_param_allocation=skip_weight_param_allocation,
                         tp_comm_buffer_name=tp_comm_buffer_name, tp_group=tp_group, stride=stride)
        self._init_fp8()

    def forward(self, input_, weight=None, runtime_gather_output=None):
        if not fp8_enabled():
            return super().forward(input_, weight, runtime_gather_output)
        w = self.weight if weight is None else weight
        x = input_
        if self.world > 1:
            x = M.gather_from_sequence_parallel_region(x, True, self.tp_group) if self.sequence_parallel \
                else M.copy_to_tensor_model_parallel_region(x, self.tp_group)
        y = fp8_linear(x, w, self)
        if self.bias is not None and not self.skip_bias_add:
            y = y + self.bias
        gather = self.gather_output if runtime_gather_output is None else runtime_gather_output
        if gather and self.world > 1:
            y = M.gather_from_tensor_model_parallel_region(y, self.tp_group)
        return y, (self.bias if self.skip_bias_add else None)


class TERowParallelLinear(RowParallelLinear, _Fp8Mixin):
    def __init__(self, input_size, output_size, *, config, init_method, bias=True, input_is_parallel=True, skip_bias_add=False,
                 is_expert=False, tp_comm_buffer_name=None, tp_group=None, stride=1, **_):
        super().__init__(input_size, output_size, config=config, init_method=init_method, bias=bias,
                         input_is_parallel=input_is_parallel, skip_bias_add=skip_bias_add, is_expert=is_expert,
                         tp_comm_buffer_name=tp_comm_buffer_name, tp_group=tp_group, stride=stride)
        self._init_fp8()

    def forward(self, input_):
        if not fp8_enabled():
            return super().forward(input_)
        x = input_ if self.input_is_parallel else M.scatter_to_tensor_model_parallel_region(input_, self.tp_group)
        y = fp8_linear(x, self.weight, self)
        if self.world > 1 and not self.explicit_expert_comm:
            y = M.reduce_scatter_to_sequence_parallel_region(y, self.tp_group) if self.sequence_parallel \
                else M.reduce_from_tensor_model_parallel_region(y, self.tp_group)
        if self.skip_bias_add:
            return y, self.bias
        return (y + self.bias if self.bias is not None else y), None


class TELayerNormColumnParallelLinear(nn.Module):
    """norm(x) -> column-parallel linear; returns (output, bias) like the Megatron spec class."""

    def __init__(self, input_size, output_size, *, config, init_method, gather_output=False, bias=True, skip_bias_add=False,
                 is_expert=False, skip_weight_param_allocation=False, tp_comm_buffer_name=None, **_):
        super().__init__()
        self.layer_norm = build_norm(config, input_size)
        self.linear = TEColumnParallelLinear(input_size, output_size, config=config, init_method=init_method,
                                             gather_output=gather_output, bias=bias, skip_bias_add=skip_bias_add,
                                             is_expert=is_expert, tp_comm_buffer_name=tp_comm_buffer_name)
        self.return_layernorm_output = False

    @property
    def weight(self):
        return self.linear.weight

    @property
    def layer_norm_weight(self):
        return self.layer_norm.weight

    def forward(self, x):
        ln = self.layer_norm(x)
        y, b = self.linear(ln)
        if self.return_layernorm_output:
            return (y, ln), b
        return y, b


class TEGroupedLinear(nn.Module, _Fp8Mixin):
    """``num_gemms`` independent linears applied to consecutive row groups (one per local expert)."""

    def __init__(self, num_gemms, input_size, output_size, *, config, init_method=None, bias=False, **_):
        super().__init__()
        if bias:
            raise NotImplementedError("grouped linears carry no bias")
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.num_gemms, self.input_size, self.output_size = num_gemms, input_size, output_size
        self.weight = nn.Parameter(torch.empty(num_gemms, output_size, input_size, device=dev, dtype=config.params_dtype))
        with torch.no_grad():
            for g in range(num_gemms):
                (init_method or config.init_method)(self.weight[g])
        setattr(self.weight, "allreduce", False)
        self._init_fp8()

    def forward(self, x, m_splits):
        counts = [int(c) for c in (m_splits.tolist() if torch.is_tensor(m_splits) else m_splits)]
        if fp8_enabled() and isinstance(_FP8State.recipe, BlockwiseScaling) and self.input_size % 128 == 0 and self.output_size % 128 == 0 \
                and not torch.is_grad_enabled():
            xq, xs = Q.quant_1x128(x)
            if "wq" not in self._fp8_wcache:
                qs = [Q.quant_128x128(self.weight[g].detach()) for g in range(self.num_gemms)]
                self._fp8_wcache.update(wq=torch.stack([q[0] for q in qs]), ws=torch.stack([q[1] for q in qs]))
            return fp8_grouped_gemm(xq, xs, self._fp8_wcache["wq"], self._fp8_wcache["ws"], counts, out_dtype=x.dtype), None
        if fp8_enabled():
            outs, s = [], 0
            for g, c in enumerate(counts):
                outs.append(fp8_linear(x[s:s + c], self.weight[g], None, _FP8State.recipe) if c else x.new_zeros(0, self.output_size))
                s += c
            return torch.cat(outs), None
        return grouped_gemm(x, self.weight.transpose(1, 2), counts, trans_b=False), None


class TEDotProductAttention(nn.Module):
    def __init__(self, config, layer_number, attn_mask_type="causal", attention_type="self", attention_dropout=None, **_):
        super().__init__()
        from .attention import CoreAttention
        self.core = CoreAttention(config, layer_number, attn_mask_type=attn_mask_type)

    def forward(self, query, key, value, attention_mask=None, attn_mask_type=None, packed_seq_params=None, **kw):
        return self.core(query, key, value, attention_mask, packed_seq_params=packed_seq_params)


class TENorm:
    def __new__(cls, config, hidden_size, eps=1e-5):
        return build_norm(config, hidden_size, eps)


class Fp8Linear(nn.Linear, _Fp8Mixin):
    """Drop-in ``nn.Linear`` whose matmul runs under a fixed recipe (used by the Megatron-free engine)."""

    def __init__(self, lin: nn.Linear, recipe: Recipe):
        nn.Module.__init__(self)
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.weight, self.bias = lin.weight, lin.bias
        self.recipe = recipe
        self._init_fp8()

    def forward(self, x):
        y = fp8_linear(x, self.weight, self, self.recipe)
        return y if self.bias is None else y + self.bias


def quantize_linears(model: nn.Module, recipe="blockwise", skip=("lm_head", "head", "embed")) -> int:
    """Replace every ``nn.Linear`` (except names containing a ``skip`` fragment) with ``Fp8Linear``."""
    rec = RECIPES[recipe]() if isinstance(recipe, str) else recipe
    n = 0
    for name, mod in list(model.named_modules()):
        if type(mod) is not nn.Linear or any(s in name for s in skip):
            continue
        parent = model
        parts = name.split(".")
        for p in parts[:-1]:
            parent = getattr(parent, p)
        setattr(parent, parts[-1], Fp8Linear(mod, rec))
        n += 1
    return n
