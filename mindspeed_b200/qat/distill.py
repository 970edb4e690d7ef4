"""Quantisation-aware distillation: a frozen full-precision teacher guides the fake-quantised student.

``TeacherManager`` owns the teacher (eval mode, no grad, optionally offloaded to host between steps) and caches its
logits for the current micro-batch; ``distillation_loss`` mixes the task loss with a temperature-scaled KL term
(and, optionally, an MSE term on chosen hidden states).  With vocab-parallel logits the softmax normalisers are
all-reduced over the tensor-parallel group so the KL is exact.
reference: mindspeed/core/distill/* (teacher manager, KL loss).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn


@dataclasses.dataclass
class DistillConfig:
    temperature: float = 1.0
    kl_weight: float = 1.0
    task_weight: float = 0.0
    hidden_mse_weight: float = 0.0
    offload_teacher: bool = False


class TeacherManager:
    def __init__(self, teacher: nn.Module, cfg: DistillConfig):
        self.teacher, self.cfg = teacher, cfg
        self.teacher.eval()
        for p in self.teacher.parameters():
            p.requires_grad_(False)
        self._home = next(teacher.parameters()).device if any(True for _ in teacher.parameters()) else torch.device("cpu")
        self._cache = None

    @torch.no_grad()
    def forward(self, *args, **kw):
        if self.cfg.offload_teacher and self._home.type == "cuda":
            self.teacher.to(self._home)
        out = self.teacher(*args, **kw)
        if self.cfg.offload_teacher and self._home.type == "cuda":
            self.teacher.to("cpu")
        self._cache = out
        return out

    def cached(self):
        return self._cache


def _log_softmax_vocab_parallel(logits, group):
    mx = logits.float().amax(-1, keepdim=True)
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    z = logits.float() - mx
    se = z.exp().sum(-1, keepdim=True)
    if group is not None and dist.get_world_size(group) > 1:
        se = _AllReduceSum.apply(se, group)
    return z - se.log()


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def distillation_loss(student_logits, teacher_logits, cfg: DistillConfig, task_loss: Optional[torch.Tensor] = None,
                      loss_mask: Optional[torch.Tensor] = None, student_hidden=None, teacher_hidden=None, tp_group=None):
    """KL(teacher || student) at temperature T, scaled by T^2, averaged over unmasked tokens."""
    T = cfg.temperature
    ls = _log_softmax_vocab_parallel(student_logits / T, tp_group)
    with torch.no_grad():
        lt = _log_softmax_vocab_parallel(teacher_logits / T, tp_group)
    kl = (lt.exp() * (lt - ls)).sum(-1)
    if tp_group is not None and dist.get_world_size(tp_group) > 1:
        kl = _AllReduceSum.apply(kl, tp_group)
    if loss_mask is not None:
        m = loss_mask.to(kl.dtype).reshape(kl.shape)
        kl = (kl * m).sum() / m.sum().clamp_min(1.0)
    else:
        kl = kl.mean()
    total = cfg.kl_weight * (T * T) * kl
    if cfg.task_weight and task_loss is not None:
        total = total + cfg.task_weight * task_loss
    if cfg.hidden_mse_weight and student_hidden is not None and teacher_hidden is not None:
        total = total + cfg.hidden_mse_weight * torch.nn.functional.mse_loss(student_hidden.float(), teacher_hidden.detach().float())
    return total
