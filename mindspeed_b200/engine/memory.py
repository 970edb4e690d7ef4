"""Memory plan of the engine: activations and optimizer state parked in pinned host memory.

``swap_activations(model, patterns)``: the forward of every matched module runs inside ``memory.host_offload.OffloadSaved``,
so what autograd saves there is copied to the host on a side stream and fetched back when backward reaches it.
``HostStateOptimizer(optimizer)``: between steps every state tensor of the wrapped optimizer lives in pinned host memory; a
step brings the state of a slice of parameters to the device (``chunk_bytes`` at a time), updates those parameters with the
wrapped optimizer's own rule and sends the state back, so the device holds one slice of state at any moment.  The two
directions are pluggable (``to_host`` / ``to_device``), which is also how the CPU tests observe the traffic.
reference: mindspeed/fsdp/memory/swap_activation/tensor_swap_manager.py, mindspeed/fsdp/memory/swap_optimizer/swap_optimizer.py.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.nn as nn

from ..memory.host_offload import OffloadSaved
from ..utils.patterns import match as _match


def swap_activations(model: nn.Module, patterns: List[str], min_bytes: int = 1 << 20, context: Optional[Callable] = None) -> int:
    """Wrap the forward of modules whose qualified name (or class name) matches; returns how many were wrapped."""
    ctx = context or (lambda: OffloadSaved(min_bytes=min_bytes))
    n = 0
    for name, mod in model.named_modules():
        if not name or getattr(mod, "_swap_wrapped", False):
            continue
        if not any(_match(name, p) or type(mod).__name__ == p for p in patterns):
            continue
        inner = mod.forward

        def forward(*a, _inner=inner, **kw):
            if not torch.is_grad_enabled():
                return _inner(*a, **kw)
            with ctx():
                return _inner(*a, **kw)
        mod.forward = forward
        mod._swap_wrapped = True
        n += 1
    return n


def _pinned_like(t: torch.Tensor) -> torch.Tensor:
    pin = torch.cuda.is_available()
    return torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)


class HostStateOptimizer:
    """Wraps a ``torch.optim.Optimizer`` whose per-parameter state tensors are to live on the host."""

    def __init__(self, optimizer: torch.optim.Optimizer, chunk_bytes: int = 256 << 20,
                 to_host: Optional[Callable] = None, to_device: Optional[Callable] = None):
        self.opt, self.chunk_bytes = optimizer, max(1, int(chunk_bytes))
        self.to_host = to_host or self._default_to_host
        self.to_device = to_device or (lambda host, like: host.to(like.device, non_blocking=True))
        self.param_groups = optimizer.param_groups
        self.moved_bytes = 0

    @staticmethod
    def _default_to_host(t: torch.Tensor) -> torch.Tensor:
        if not t.is_cuda:
            return t
        h = _pinned_like(t)
        h.copy_(t, non_blocking=True)
        return h

    def _slices(self):
        """Lists of parameters whose state fits ``chunk_bytes`` (2 moment tensors per parameter assumed until state exists)."""
        cur, size = [], 0
        for g in self.opt.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                b = 2 * p.numel() * max(4, p.element_size())
                if cur and size + b > self.chunk_bytes:
                    yield cur
                    cur, size = [], 0
                cur.append(p)
                size += b
        if cur:
            yield cur

    def _fetch(self, params):
        for p in params:
            for k, v in self.opt.state.get(p, {}).items():
                if torch.is_tensor(v) and v.numel() > 1 and getattr(v, "_on_host", False):
                    d = self.to_device(v, p)
                    self.moved_bytes += v.numel() * v.element_size()
                    self.opt.state[p][k] = d

    def _park(self, params):
        for p in params:
            for k, v in self.opt.state.get(p, {}).items():
                if torch.is_tensor(v) and v.numel() > 1:
                    h = self.to_host(v)
                    h._on_host = True
                    self.moved_bytes += v.numel() * v.element_size()
                    self.opt.state[p][k] = h

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for params in self._slices():
            self._fetch(params)
            keep = {}
            wanted = {id(p) for p in params}
            for g in self.opt.param_groups:          # hide the gradients of the other slices: the wrapped step skips them
                for p in g["params"]:
                    if id(p) not in wanted and p.grad is not None:
                        keep[p] = p.grad
                        p.grad = None
            try:
                self.opt.step()
            finally:
                for p, gr in keep.items():
                    p.grad = gr
            self._park(params)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()     # host copies are complete before the buffers are reused
        return loss

    def zero_grad(self, set_to_none: bool = True):
        self.opt.zero_grad(set_to_none)

    def state_dict(self):
        return self.opt.state_dict()

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd)
        for g in self.opt.param_groups:
            self._park(g["params"])
