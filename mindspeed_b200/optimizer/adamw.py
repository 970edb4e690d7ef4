"""Per-parameter AdamW (the optimizer the reference installs in place of apex FusedAdam).

Semantics follow ``torch._fused_adamw_`` with decoupled weight decay and an integer step kept in the
param group (reference: mindspeed/core/optimizer/adamw.py:9-20,96-189).  On a GPU each parameter is
updated by the flat fused kernel (one launch per tensor); on CPU by the eager restatement.
"""
from __future__ import annotations

import torch
from torch.optim.optimizer import Optimizer

from ..ops.adam import adam_flat


class AdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False, *,
                 maximize: bool = False, bias_correction: bool = True, adam_w_mode: bool = True, **_unused):
        if amsgrad:
            raise ValueError("amsgrad is not supported by the fused kernel")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, maximize=maximize, step=0,
                        bias_correction=bias_correction, adam_w_mode=adam_w_mode)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            group["step"] = group.get("step", 0) + 1
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                if p.dtype == torch.float32 and p.is_contiguous():
                    adam_flat(p.data.view(-1), p.grad.contiguous().view(-1), st["exp_avg"].view(-1),
                              st["exp_avg_sq"].view(-1), None, group["lr"], b1, b2, group["eps"], group["weight_decay"],
                              group["step"], 1.0, group["adam_w_mode"], bias_correction=group["bias_correction"],
                              maximize=group["maximize"])
                else:
                    if "master" not in st:
                        st["master"] = p.data.float().contiguous()
                    adam_flat(st["master"].view(-1), p.grad.contiguous().view(-1), st["exp_avg"].view(-1),
                              st["exp_avg_sq"].view(-1), None, group["lr"], b1, b2, group["eps"], group["weight_decay"],
                              group["step"], 1.0, group["adam_w_mode"], bias_correction=group["bias_correction"],
                              maximize=group["maximize"])
                    p.data.copy_(st["master"])
        return loss


class FusedTorchAdamW(torch.optim.AdamW):
    """``--optimizer-selection fused_torch_adamw``: torch's own fused implementation."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **kw):
        fused = torch.cuda.is_available()
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=fused)
