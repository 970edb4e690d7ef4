"""Top-1 / top-2 gating with capacity (GShard / DeepSpeed formulation)."""
from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _capacity(tokens: int, experts: int, factor: float, min_capacity: int) -> int:
    return max(min_capacity, int(math.ceil(tokens / experts * factor)))


def _locations(mask):
    """Position of every token inside its expert's buffer: exclusive running count down the token dimension."""
    return torch.cumsum(mask, dim=0) - mask


def top1gating(logits, capacity_factor=1.0, min_capacity=4, noisy_gate_policy=None, use_rts=False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """logits [S, E] -> (aux loss, combine weights [S, E, C], dispatch mask [S, E, C] bool, tokens per expert [E]).
    ``use_rts`` (random token selection): when an expert is over capacity the tokens it keeps are drawn at random instead
    of being the first ones in sequence order, which removes the bias towards early positions."""
    S, E = logits.shape
    gates = F.softmax(logits.float(), dim=1)
    C = _capacity(S, E, capacity_factor, min_capacity)
    sel = logits + torch.randn_like(logits) * 1e-2 if noisy_gate_policy == "RSample" else logits
    idx = sel.argmax(dim=1)
    mask = F.one_hot(idx, E).to(gates.dtype)
    exp_counts = mask.sum(0).detach()
    me, ce = gates.mean(0), mask.mean(0)
    l_aux = (me * ce).sum() * E
    if use_rts:
        prio = mask * torch.rand_like(mask)                      # a random priority for every (token, chosen expert)
        keep = torch.zeros_like(mask)
        top = torch.topk(prio, k=min(C, S), dim=0).indices       # per expert: its C highest priorities
        keep.scatter_(0, top, 1.0)
        mask = mask * keep
        loc = _locations(mask)
    else:
        loc = _locations(mask)
        mask = mask * (loc < C)
    loc_s = (loc * mask).sum(1).long()
    gate_s = (gates * mask).sum(1)
    combine = gate_s.view(S, 1, 1) * mask.unsqueeze(-1) * F.one_hot(loc_s, C).to(gates.dtype).unsqueeze(1)
    return l_aux, combine, combine.bool(), exp_counts


def top2gating(logits, capacity_factor=1.0, min_capacity=4) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    S, E = logits.shape
    gates = F.softmax(logits.float(), dim=1)
    C = _capacity(S, E, 2 * capacity_factor, min_capacity)
    idx1 = gates.argmax(dim=1)
    mask1 = F.one_hot(idx1, E).to(gates.dtype)
    idx2 = gates.masked_fill(mask1.bool(), float("-inf")).argmax(dim=1)
    mask2 = F.one_hot(idx2, E).to(gates.dtype)
    loc1 = _locations(mask1)
    loc2 = _locations(mask2) + mask1.sum(0, keepdim=True)       # second choices queue behind all first choices
    exp_counts = (mask1 + mask2).sum(0).detach()
    me, ce = gates.mean(0), mask1.mean(0)
    l_aux = (me * ce).sum() * E
    mask1 = mask1 * (loc1 < C)
    mask2 = mask2 * (loc2 < C)
    l1, l2 = (loc1 * mask1).sum(1).long(), (loc2 * mask2).sum(1).long()
    g1, g2 = (gates * mask1).sum(1), (gates * mask2).sum(1)
    den = (g1 + g2).clamp_min(torch.finfo(gates.dtype).eps)
    g1, g2 = g1 / den, g2 / den
    c1 = g1.view(S, 1, 1) * mask1.unsqueeze(-1) * F.one_hot(l1, C).to(gates.dtype).unsqueeze(1)
    c2 = g2.view(S, 1, 1) * mask2.unsqueeze(-1) * F.one_hot(l2, C).to(gates.dtype).unsqueeze(1)
    combine = c1 + c2
    return l_aux, combine, combine.bool(), exp_counts


class TopKGate(nn.Module):
    def __init__(self, model_dim, num_experts, k=1, capacity_factor=1.0, eval_capacity_factor=1.0, min_capacity=4,
                 noisy_gate_policy=None, use_rts=False):
        super().__init__()
        self.use_rts = use_rts
        if k not in (1, 2):
            raise ValueError("only top-1 and top-2 gating are supported")
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.k, self.cf, self.ecf, self.min_capacity, self.noisy = k, capacity_factor, eval_capacity_factor, min_capacity, noisy_gate_policy

    def forward(self, x):
        logits = self.wg(x.float())
        cf = self.cf if self.training else self.ecf
        if self.k == 1:
            return top1gating(logits, cf, self.min_capacity, self.noisy if self.training else None, self.use_rts and self.training)
        return top2gating(logits, cf, self.min_capacity)
