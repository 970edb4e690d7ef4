"""Quantisation-aware distillation wired into training (``--qad-enable``).

A second copy of the model - the teacher - is built from the same provider, loaded from ``--qad-teacher-load``, frozen and
kept in evaluation mode without fake quantisation; the student is the model being trained (with ``--qat-scheme`` its
linears run on fake-quantised weights).  Every micro-batch the teacher's logits are computed without a graph from the same
tokens, and the student is trained on the KL divergence from the teacher's distribution alone: temperature
``--kl-temperature`` (loss scaled by T^2), weight ``--kl-loss-weight``, ``--kl-loss-reduction`` mean (over unmasked
tokens) or sum.  The cross entropy against the labels is computed without a graph and reported next to it.  With
vocabulary-parallel logits the softmax normalisers are reduced over the tensor-parallel group, so the loss equals the
single-rank one.  Dense models without pipeline parallelism only: the loss needs both models' logits for the same
micro-batch on one rank.

reference: mindspeed/features_manager/qad/qad_quant_engine.py:17-175, mindspeed/core/distill/qad_adapter.py,
mindspeed/core/distill/teacher_model_manager.py, mindspeed/core/distill/logits_kl_loss.py:15-164.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .distill import DistillConfig, TeacherManager, _AllReduceSum, _log_softmax_vocab_parallel

_TEACHER = None


def get_teacher():
    if _TEACHER is None:
        raise RuntimeError("--qad-enable: the teacher has not been built (setup_teacher runs in setup_model_and_optimizer)")
    return _TEACHER


def reset():
    global _TEACHER
    _TEACHER = None


def load_model_weights(model, load_dir, iteration=None, strict=True):
    """Model weights only (no optimizer, scheduler or RNG state) of a checkpoint directory into ``model`` (list of chunks)."""
    from .. import checkpointing as C
    it = iteration if iteration is not None else C.read_latest_iteration(load_dir)
    if it is None:
        raise FileNotFoundError(f"no checkpoint under {load_dir!r} (latest_checkpointed_iteration.txt is missing)")
    sharded, _ = C.generate_state_dict(model, None, None, it, None, rng=False)
    missing = C._load_sharded(sharded, C.get_checkpoint_name(load_dir, it), strict=False)
    if strict and missing:
        # persistent buffers (rotary frequencies and the like) are rebuilt by the model and may be absent from converted
        # checkpoints; a missing parameter is an error
        buffers = set()
        for chunk in model:
            inner = chunk.module if hasattr(chunk, "module") and not hasattr(chunk, "decoder") else chunk
            buffers.update(n for n, _ in inner.named_buffers())
        bad = [k for k in missing if k.split("@")[0] not in buffers]
        if bad:
            raise KeyError(f"keys missing from checkpoint: {bad[:5]} ...")
    return it


def setup_teacher(model_provider_func, args):
    """Build, load and freeze the teacher.  Called once, after the student exists and before the first step."""
    global _TEACHER
    from ..training.training import get_model
    chunks = get_model(model_provider_func, wrap_with_ddp=False)
    if len(chunks) != 1:
        raise AssertionError("--qad-enable needs the whole model on one pipeline stage")
    load_model_weights(chunks, args.qad_teacher_load)
    _TEACHER = TeacherManager(chunks[0], DistillConfig(temperature=args.kl_temperature, kl_weight=args.kl_loss_weight))
    return _TEACHER


def kl_from_logits(student_logits, teacher_logits, loss_mask=None, temperature=1.0, reduction="mean", tp_group=None):
    """KL(teacher || student) * T^2 from (vocabulary-parallel) logits ``[..., V / tp]``; ``loss_mask`` selects tokens."""
    T = float(temperature)
    ls = _log_softmax_vocab_parallel(student_logits / T, tp_group)
    with torch.no_grad():
        lt = _log_softmax_vocab_parallel(teacher_logits / T, tp_group)
    kl = (lt.exp() * (lt - ls)).sum(-1)
    if tp_group is not None and dist.get_world_size(tp_group) > 1:
        kl = _AllReduceSum.apply(kl, tp_group)
    kl = kl * (T * T)
    m = torch.ones_like(kl) if loss_mask is None else loss_mask.to(kl.dtype).reshape(kl.shape)
    total, n = (kl * m).sum(), m.sum()
    if reduction == "sum":
        return total, n
    if reduction == "mean":
        return total / n.clamp_min(1.0), n
    raise ValueError("--kl-loss-reduction is mean or sum")


def qad_loss_func(loss_mask, labels, teacher_logits, args, student_logits):
    """Loss function of one micro-batch (last argument: the student's output, as the schedules call it)."""
    from ..parallel import parallel_state as ps
    from ..parallel.cross_entropy import vocab_parallel_cross_entropy
    tp_group = ps.get_tensor_model_parallel_group() if ps.get_tensor_model_parallel_world_size() > 1 else None
    kl, n = kl_from_logits(student_logits, teacher_logits, loss_mask, args.kl_temperature, args.kl_loss_reduction, tp_group)
    loss = args.kl_loss_weight * kl
    with torch.no_grad():
        ce = vocab_parallel_cross_entropy(student_logits.detach().transpose(0, 1).float().contiguous(),
                                          labels.transpose(0, 1).contiguous()).transpose(0, 1)
        m = loss_mask.reshape(ce.shape).float()
        # reported as [numerator, denominator] pairs, summed over data-parallel ranks and micro-batches before dividing:
        # token-weighted means; with reduction "sum" the KL entry is the mean of the per-micro-batch sums
        mean = args.kl_loss_reduction == "mean"
        rep = torch.stack([(ce * m).sum(), m.sum(), kl.detach() * (n if mean else 1.0), n if mean else torch.ones_like(n)])
        dist.all_reduce(rep, group=ps.get_data_parallel_group())
    return loss, {"lm loss": rep[:2].clone(), "kl loss": rep[2:].clone()}


def qad_forward_step(tokens, labels, loss_mask, attention_mask, position_ids, packed, model, args):
    """Teacher (no graph) and student forward of one micro-batch; returns (student logits, loss function)."""
    from functools import partial
    teacher_logits = get_teacher().forward(tokens, position_ids, attention_mask, packed_seq_params=packed)
    out = model(tokens, position_ids, attention_mask, packed_seq_params=packed)
    return out, partial(qad_loss_func, loss_mask, labels, teacher_logits, args)
