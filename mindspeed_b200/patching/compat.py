"""Stand-ins for optional native packages that Megatron-style training scripts import unconditionally
(``apex``, ``amp_C``, ``fused_layer_norm_cuda``, ``transformer_engine``, ``flash_attn``), mapped onto this framework's own
ops, plus two small helpers such scripts expect from the training utilities.

``optional_dependency_stubs()`` lists ``(dotted path, object)`` pairs; the adaptor installs a pair only when the package
named by the path's first component cannot be imported, so an installed apex / flash-attn / Transformer Engine is never
shadowed.

  amp_C.multi_tensor_l2norm / _scale / _axpby / _adam     chunked multi-tensor functors with apex's calling convention
                                                          (``op(chunk_size, noop_flag, tensor_lists, *args)``); the noop
                                                          flag is set when a non-finite value is met, as apex does
  apex.multi_tensor_apply.multi_tensor_applier            calls the functor
  apex.optimizers.FusedAdam / FusedSGD                    torch AdamW / SGD (fused implementation on CUDA)
  apex.normalization.FusedLayerNorm / FusedRMSNorm / MixedFusedRMSNorm      this framework's norm modules (own kernels on CUDA)
  transformer_engine.pytorch.{Linear, LayerNorm, RMSNorm, LayerNormLinear, GroupedLinear, DotProductAttention, fp8_autocast}
  transformer_engine.common.recipe.{DelayedScaling, Format}                 ``models/te_compat.py``
  flash_attn.flash_attn_interface.flash_attn_func / flash_attn_varlen_func / flash_attn_unpadded_func
                                                          ``ops/attention.py`` ([b, s, h, d] / packed [t, h, d] layouts)
reference: mindspeed/features_manager/megatron_basic/requirements_basic.py:32-115 (the same set of stand-ins for its device),
mindspeed/core/megatron_basic/requirements_basic.py:7-100.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch


# ----------------------------------------------------------------------------------------------------------------------
# amp_C / apex.multi_tensor_apply
# ----------------------------------------------------------------------------------------------------------------------
def multi_tensor_applier(op, noop_flag, tensor_lists, *args):
    return op(2048 * 32, noop_flag, tensor_lists, *args)


def _flag(noop_flag, tensors: Sequence[torch.Tensor]):
    """Set the overflow flag when any tensor holds a non-finite value (checked with one fused reduction per list)."""
    if not torch.is_tensor(noop_flag) or not tensors:
        return
    bad = torch.stack([(~torch.isfinite(t)).any() for t in tensors]).any()
    noop_flag.copy_(torch.maximum(noop_flag.to(torch.int32), bad.to(torch.int32).reshape(noop_flag.shape)).to(noop_flag.dtype))


def multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor=False, *_):
    ts = tensor_lists[0]
    dev = ts[0].device if ts else (noop_flag.device if torch.is_tensor(noop_flag) else "cpu")
    if not ts:
        return torch.zeros(1, device=dev), (torch.zeros(0, device=dev) if per_tensor else None)
    norms = torch.stack(torch._foreach_norm([t.float() for t in ts], 2)) if hasattr(torch, "_foreach_norm") \
        else torch.stack([t.float().norm(2) for t in ts])
    return norms.norm(2).reshape(1), (norms if per_tensor else None)


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    src, dst = tensor_lists
    _flag(noop_flag, src)
    for s, d in zip(src, dst):
        d.copy_(s * scale)


def multi_tensor_axpby(chunk_size, noop_flag, tensor_lists, a, b, arg_to_check=-1):
    """out = a * x + b * y; ``arg_to_check`` 0 / 1 / -1: which input (x, y, both) feeds the overflow flag."""
    xs, ys, outs = tensor_lists
    _flag(noop_flag, (list(xs) if arg_to_check in (-1, 0) else []) + (list(ys) if arg_to_check in (-1, 1) else []))
    for x, y, o in zip(xs, ys, outs):
        o.copy_(a * x.float() + b * y.float())


def multi_tensor_adam(chunk_size, noop_flag, tensor_lists, lr, beta1, beta2, eps, step, mode, bias_correction, weight_decay):
    """Adam over lists [grads, params, exp_avgs, exp_avg_sqs]; ``mode`` 0 = L2 regularisation, 1 = decoupled weight decay."""
    gs, ps, ms, vs = tensor_lists
    c1 = 1.0 - beta1 ** step if bias_correction else 1.0
    c2 = 1.0 - beta2 ** step if bias_correction else 1.0
    for g, p, m, v in zip(gs, ps, ms, vs):
        gf = g.float()
        if mode == 0 and weight_decay:
            gf = gf + weight_decay * p.float()
        m.mul_(beta1).add_(gf.to(m.dtype), alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gf.to(v.dtype), gf.to(v.dtype), value=1 - beta2)
        upd = (m.float() / c1) / ((v.float() / c2).sqrt() + eps)
        if mode == 1 and weight_decay:
            upd = upd + weight_decay * p.float()
        p.add_((-lr * upd).to(p.dtype))


# ----------------------------------------------------------------------------------------------------------------------
# apex.optimizers / apex.normalization
# ----------------------------------------------------------------------------------------------------------------------
class FusedAdamStub(torch.optim.AdamW):
    """``apex.optimizers.FusedAdam(params, lr, betas, eps, weight_decay, adam_w_mode=True)`` on torch's fused AdamW."""

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True, weight_decay=0.0,
                 amsgrad=False, set_grad_none=True, **_):
        if not adam_w_mode:
            raise NotImplementedError("L2-regularised (non-decoupled) Adam is not provided")
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)


class FusedSGDStub(torch.optim.SGD):
    """``apex.optimizers.FusedSGD``: torch SGD; apex-only keywords are accepted and ignored."""

    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, wd_after_momentum=False,
                 materialize_master_grads=True, set_grad_none=False, **_):
        super().__init__(params, lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)


def _norm_classes():
    from ..models.norms import LayerNorm, RMSNorm

    class FusedLayerNorm(LayerNorm):
        def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, **_):
            n = normalized_shape if isinstance(normalized_shape, int) else math.prod(normalized_shape)
            super().__init__(n, eps=eps)

    class FusedRMSNorm(RMSNorm):
        def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, **_):
            n = normalized_shape if isinstance(normalized_shape, int) else math.prod(normalized_shape)
            super().__init__(n, eps=eps)
    return FusedLayerNorm, FusedRMSNorm


# ----------------------------------------------------------------------------------------------------------------------
# flash_attn.flash_attn_interface
# ----------------------------------------------------------------------------------------------------------------------
def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, **_):
    """q, k, v [b, s, h, d] -> [b, s, h, d]."""
    from ..ops.attention import flash_attention
    if dropout_p:
        raise NotImplementedError("attention dropout is applied by the caller in this framework")
    o = flash_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), causal=causal, softmax_scale=softmax_scale)
    return o.transpose(0, 1)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None, max_seqlen_k=None, dropout_p=0.0,
                           softmax_scale=None, causal=False, **_):
    """Packed layout: q, k, v [total tokens, h, d] with the sequences' boundaries in ``cu_seqlens_*`` (self attention:
    both boundary lists are the same)."""
    from ..ops.attention import varlen_attention
    if dropout_p:
        raise NotImplementedError("attention dropout is applied by the caller in this framework")
    cq = cu_seqlens_q.tolist() if torch.is_tensor(cu_seqlens_q) else list(cu_seqlens_q)
    ck = cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else list(cu_seqlens_k)
    if cq != ck:
        raise NotImplementedError("packed attention with different query and key boundaries")
    o = varlen_attention(q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1), cq, causal=causal, softmax_scale=softmax_scale)
    return o.squeeze(1)


# ----------------------------------------------------------------------------------------------------------------------
# training utilities
# ----------------------------------------------------------------------------------------------------------------------
def count_zeros_fp32(parameters, grad_stats_parallel_group=None, use_main_grad: bool = True) -> float:
    """Number of exactly-zero gradient entries over ``parameters``, each shared / tensor-parallel-duplicated parameter counted
    once, summed over ``grad_stats_parallel_group`` (the model-parallel group).  Reads ``main_grad`` when the parameter has
    one (the distributed-data-parallel buffers), else ``grad``."""
    import torch.distributed as dist
    from ..parallel import parallel_state as ps
    if torch.is_tensor(parameters):
        parameters = [parameters]
    total = None
    for p in parameters:
        g = getattr(p, "main_grad", None) if use_main_grad else None
        g = p.grad if g is None else g
        if g is None:
            continue
        dup = getattr(p, "shared", False) or (not getattr(p, "tensor_model_parallel", False)
                                              and ps.model_parallel_is_initialized() and ps.get_tensor_model_parallel_rank() != 0)
        if dup:
            continue
        z = (g.numel() - torch.count_nonzero(g)).float()
        total = z if total is None else total + z
    if total is None:
        total = torch.zeros(())
    if grad_stats_parallel_group is not None and dist.is_initialized():
        total = total.clone()
        dist.all_reduce(total, group=grad_stats_parallel_group)
    return float(total)


def optional_dependency_stubs() -> List[tuple]:
    from ..models import te_compat as TE
    FusedLayerNorm, FusedRMSNorm = _norm_classes()

    class _Format:
        E4M3, HYBRID = "e4m3", "hybrid"

    class TELinear(TE.Fp8Linear):
        """``transformer_engine.pytorch.Linear(in_features, out_features, bias=True)``: fp8 under ``fp8_autocast``."""

        def __init__(self, in_features, out_features, bias=True, params_dtype=None, device=None, **_):
            super().__init__(torch.nn.Linear(in_features, out_features, bias=bias, device=device, dtype=params_dtype), None)

        def forward(self, x):
            if not TE.fp8_enabled():
                return torch.nn.functional.linear(x, self.weight, self.bias)
            return super().forward(x)
    return [
        ("amp_C.multi_tensor_l2norm", multi_tensor_l2norm),
        ("amp_C.multi_tensor_scale", multi_tensor_scale),
        ("amp_C.multi_tensor_axpby", multi_tensor_axpby),
        ("amp_C.multi_tensor_adam", multi_tensor_adam),
        ("apex.multi_tensor_apply.multi_tensor_applier", multi_tensor_applier),
        ("apex.optimizers.FusedAdam", FusedAdamStub),
        ("apex.optimizers.FusedSGD", FusedSGDStub),
        ("apex.normalization.FusedLayerNorm", FusedLayerNorm),
        ("apex.normalization.FusedRMSNorm", FusedRMSNorm),
        ("apex.normalization.MixedFusedRMSNorm", FusedRMSNorm),
        ("fused_layer_norm_cuda.available", True),
        ("transformer_engine.pytorch.Linear", TELinear),
        ("transformer_engine.pytorch.LayerNorm", FusedLayerNorm),
        ("transformer_engine.pytorch.RMSNorm", FusedRMSNorm),
        ("transformer_engine.pytorch.LayerNormLinear", TE.TELayerNormColumnParallelLinear),
        ("transformer_engine.pytorch.GroupedLinear", TE.TEGroupedLinear),
        ("transformer_engine.pytorch.DotProductAttention", TE.TEDotProductAttention),
        ("transformer_engine.pytorch.fp8_autocast", TE.fp8_autocast),
        ("transformer_engine.common.recipe.DelayedScaling", TE.DelayedScaling),
        ("transformer_engine.common.recipe.Format", _Format),
        ("flash_attn.flash_attn_interface.flash_attn_func", flash_attn_func),
        ("flash_attn.flash_attn_interface.flash_attn_varlen_func", flash_attn_varlen_func),
        ("flash_attn.flash_attn_interface.flash_attn_unpadded_func", flash_attn_varlen_func),
    ]
