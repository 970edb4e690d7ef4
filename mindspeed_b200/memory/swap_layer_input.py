"""Offload every transformer layer's *input* hidden state to pinned host memory and prefetch it in backward.

Combined with full recompute this removes the last per-layer activation that recompute keeps on the device: the
layer input.  Forward: after layer i has consumed its input the tensor is copied to the host on a side stream and
its device storage released; backward: when layer i+1 starts its backward, layer i's input is copied back, so the
copy hides behind layer i+1's recompute + backward.
reference: mindspeed/core/memory/swap_layer_input/swap_layer_input.py:8-120, swap_layer_input_manager.py.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn


class _SwapInput(torch.autograd.Function):
    """Identity on the layer input whose *saved* copy lives on the host."""

    @staticmethod
    def forward(ctx, x, mgr, idx):
        ctx.mgr, ctx.idx = mgr, idx
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class LayerInputSwapper:
    def __init__(self, layers: List[nn.Module], min_bytes: int = 1 << 20):
        self.layers, self.min_bytes = layers, min_bytes
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.host: Dict[int, torch.Tensor] = {}
        self.events: Dict[int, object] = {}
        self.restored: Dict[int, torch.Tensor] = {}
        self.bytes_swapped = 0
        self._handles = []
        for i, l in enumerate(layers):
            self._handles.append(l.register_forward_hook(self._after_forward(i)))
            self._handles.append(l.register_full_backward_pre_hook(self._before_backward(i)))

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    def _after_forward(self, i):
        def hook(mod, args, out):
            x = args[0] if args else None
            if not (isinstance(x, torch.Tensor) and torch.is_grad_enabled() and x.requires_grad):
                return
            nbytes = x.numel() * x.element_size()
            if nbytes < self.min_bytes:
                return
            if x.is_cuda:
                h = torch.empty(x.shape, dtype=x.dtype, device="cpu", pin_memory=True)
                self.stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.stream):
                    h.copy_(x.detach(), non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                self.events[i] = ev
            else:
                h = x.detach().clone()
            self.host[i] = h
            self.bytes_swapped += nbytes
        return hook

    def release_device_copies(self, tensors: Dict[int, torch.Tensor]):
        """Free the device storage of swapped inputs once their copies completed (call at a layer boundary with the
        tensors that only recompute will need again)."""
        for i, t in tensors.items():
            if i in self.host and t.is_cuda:
                self.events[i].synchronize()
                t.untyped_storage().resize_(0)

    def _before_backward(self, i):
        def hook(mod, grad_out):
            # prefetch the previous layer's input while this layer runs its backward
            j = i - 1
            if j in self.host and j not in self.restored and self.host[j].is_pinned():
                with torch.cuda.stream(self.stream):
                    self.restored[j] = self.host[j].to("cuda", non_blocking=True)
        return hook

    def fetch(self, i: int) -> Optional[torch.Tensor]:
        """The input of layer ``i`` on the device (waits for the prefetch); None when it was never swapped."""
        if i not in self.host:
            return None
        if i in self.restored:
            torch.cuda.current_stream().wait_stream(self.stream)
            return self.restored.pop(i)
        h = self.host[i]
        return h.to("cuda", non_blocking=True) if h.is_pinned() else h

    def reset(self):
        self.host.clear(); self.events.clear(); self.restored.clear()
