"""MOELayer: gate -> dispatch (einsum) -> all-to-all -> local experts -> all-to-all -> combine (einsum)."""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.nn as nn

from ..parallel import mappings as M
from .gate import TopKGate


class Experts(nn.Module):
    """``num_local_experts`` copies of ``expert``; input [E_local, C', H] -> same shape."""

    def __init__(self, expert: nn.Module, num_local_experts: int = 1):
        super().__init__()
        # ``expert`` is a module (copied, as DeepSpeed does) or a zero-argument factory (modules that hold process groups
        # cannot be deep-copied)
        if isinstance(expert, nn.Module):
            self.experts = nn.ModuleList([copy.deepcopy(expert) for _ in range(num_local_experts)])
        else:
            self.experts = nn.ModuleList([expert() for _ in range(num_local_experts)])
        for e in self.experts:
            for p in e.parameters():
                p.allreduce = False

    def forward(self, x):
        outs = []
        for chunk, e in zip(x.chunk(len(self.experts), dim=0), self.experts):
            o = e(chunk)
            outs.append(o[0] if isinstance(o, tuple) else o)
        return torch.cat(outs, dim=0)


class MOELayer(nn.Module):
    def __init__(self, gate: TopKGate, experts: Experts, ep_group, ep_size: int, num_local_experts: int, pipe_experts: int = 1):
        super().__init__()
        self.gate, self.experts = gate, experts
        self.ep_group, self.ep_size, self.num_local_experts = ep_group, ep_size, num_local_experts
        self.pipe_experts = max(1, pipe_experts)
        self.multi_stream = False            # chunks' all-to-alls on a second CUDA stream (--pipe-experts-multi-stream)
        self._comm_stream = None
        self.l_aux = None
        self.exp_counts = None

    def _a2a(self, x):
        if self.ep_size <= 1:
            return x
        if self.multi_stream and x.is_cuda and self.pipe_experts > 1:
            # the exchange of this chunk runs beside the expert computation of the previous one
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=x.device)
            main = torch.cuda.current_stream()
            self._comm_stream.wait_stream(main)
            x.record_stream(self._comm_stream)
            with torch.cuda.stream(self._comm_stream):
                y = M.all_to_all(self.ep_group, x)
            y.record_stream(main)
            main.wait_stream(self._comm_stream)
            return y
        return M.all_to_all(self.ep_group, x)

    def forward(self, x):
        d = x.shape[-1]
        flat = x.reshape(-1, d)
        self.l_aux, combine, dispatch, self.exp_counts = self.gate(flat)
        E, C = dispatch.shape[1], dispatch.shape[2]
        buf = torch.einsum("sec,sm->ecm", dispatch.to(flat.dtype), flat)                  # [E, C, d]
        outs = []
        # capacity chunks: each is exchanged and computed independently, so a chunk's all-to-all can overlap the
        # previous chunk's expert compute when the caller runs communication on a side stream
        for part in buf.chunk(self.pipe_experts, dim=1):
            c = part.shape[1]
            p = self._a2a(part.contiguous().view(E * c, d)).view(self.ep_size, self.num_local_experts, c, d)
            p = p.permute(1, 0, 2, 3).reshape(self.num_local_experts, self.ep_size * c, d)  # [E_loc, ep*c, d]
            y = self.experts(p)
            y = y.view(self.num_local_experts, self.ep_size, c, d).permute(1, 0, 2, 3).reshape(E * c, d)
            outs.append(self._a2a(y.contiguous()).view(E, c, d))
        y = torch.cat(outs, dim=1)
        out = torch.einsum("sec,ecm->sm", combine.to(flat.dtype), y)
        return out.view(x.shape)


class MoE(nn.Module):
    """User-facing wrapper: returns (output, auxiliary loss, tokens per expert)."""

    def __init__(self, hidden_size, expert: nn.Module, num_experts=1, ep_size=1, k=1, capacity_factor=1.0, eval_capacity_factor=1.0,
                 min_capacity=4, noisy_gate_policy: Optional[str] = None, ep_group=None, pipe_experts: int = 1, use_rts: bool = False):
        super().__init__()
        if num_experts % ep_size != 0:
            raise ValueError("num_experts must be divisible by ep_size")
        self.num_local_experts = num_experts // ep_size
        gate = TopKGate(hidden_size, num_experts, k, capacity_factor, eval_capacity_factor, min_capacity, noisy_gate_policy, use_rts)
        self.moe_layer = MOELayer(gate, Experts(expert, self.num_local_experts), ep_group, ep_size, self.num_local_experts, pipe_experts)

    def forward(self, hidden_states):
        out = self.moe_layer(hidden_states)
        return out, self.moe_layer.l_aux, self.moe_layer.exp_counts
