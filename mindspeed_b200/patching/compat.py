"""Python stand-ins for optional native extensions that training scripts import unconditionally.
reference: mindspeed/core/megatron_basic/requirements_basic.py:7-100 (amp_C multi-tensor fallbacks, FusedAdam -> AdamW)."""
from __future__ import annotations

import torch


def multi_tensor_applier(op, noop_flag, tensor_lists, *args):
    return op(2048 * 32, noop_flag, tensor_lists, *args)


def multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor=False, *_):
    ts = tensor_lists[0]
    norms = [t.float().norm(2) for t in ts]
    total = torch.stack(norms).norm(2) if norms else torch.zeros((), device=noop_flag.device if torch.is_tensor(noop_flag) else "cpu")
    return total.reshape(1), (torch.stack(norms) if per_tensor and norms else None)


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    for src, dst in zip(*tensor_lists):
        dst.copy_(src * scale)


class FusedAdamStub(torch.optim.AdamW):
    """``apex.optimizers.FusedAdam(params, lr, betas, eps, weight_decay, adam_w_mode=True)`` on torch's fused AdamW."""

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True, weight_decay=0.0,
                 amsgrad=False, set_grad_none=True, **_):
        if not adam_w_mode:
            raise NotImplementedError("L2-regularised (non-decoupled) Adam is not provided")
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
