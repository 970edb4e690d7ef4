"""Activation offload to pinned host memory with backward prefetch ("swap attention" / "swap layer input").

Tensors saved for backward inside the selected modules are copied to pinned host buffers with ``cudaMemcpyAsync`` on
a side stream as soon as they are saved; the device copy is released at the next layer boundary once the copy has
finished.  In backward, when layer i starts, the tensors of layer i-1 are copied back on the same side stream so the
transfer hides behind layer i's compute.
Selection rules follow the reference (mindspeed/core/memory/swap_attention/prefetch.py:124-130,160-184): skip tensors
under 1 MiB, tensors without grad_fn (parameters, inputs) and views are tracked by storage so a tensor saved twice is
copied once.  Which layers swap and which recompute follows ``--recompute-num-layers`` (adaptor.py:102-146).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

MIN_BYTES = 1 << 20


class _Handle:
    __slots__ = ("dev", "host", "shape", "dtype", "device", "d2h_event", "h2d_event", "layer", "stride", "offset", "key")

    def __init__(self, t, layer):
        self.dev: Optional[torch.Tensor] = t
        self.host: Optional[torch.Tensor] = None
        self.shape, self.dtype, self.device = t.shape, t.dtype, t.device
        self.d2h_event = self.h2d_event = None
        self.layer = layer


class SwapManager:
    def __init__(self, min_bytes: int = MIN_BYTES):
        self.min_bytes = min_bytes
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.layers: Dict[int, List[_Handle]] = {}
        self.by_storage: Dict[int, _Handle] = {}
        self.current_layer = -1
        self.bytes_swapped = 0
        self.enabled = True

    # ---- saved-tensor hooks ----
    def pack(self, t: torch.Tensor):
        if (not self.enabled or not t.is_cuda or t.grad_fn is None or t.numel() * t.element_size() < self.min_bytes
                or t.untyped_storage().size() == 0 or not t.is_contiguous()):
            return t
        key = (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape))
        h = self.by_storage.get(key)
        if h is not None and h.layer == self.current_layer:
            return h
        h = _Handle(t, self.current_layer)
        h.host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ev)
            h.host.copy_(t, non_blocking=True)
            h.d2h_event = torch.cuda.Event()
            h.d2h_event.record(self.stream)
        self.by_storage[key] = h
        self.layers.setdefault(self.current_layer, []).append(h)
        self.bytes_swapped += t.numel() * t.element_size()
        return h

    def unpack(self, obj):
        if not isinstance(obj, _Handle):
            return obj
        if obj.dev is None:
            self._h2d(obj)
        if obj.h2d_event is not None:
            torch.cuda.current_stream().wait_event(obj.h2d_event)
            obj.h2d_event = None
        return obj.dev

    # ---- layer boundaries ----
    def release_device_copies(self, layer: int):
        """Called when a later layer starts its forward: the copies of ``layer`` are done, drop the device side."""
        for h in self.layers.get(layer, []):
            if h.dev is not None and h.d2h_event is not None:
                h.d2h_event.synchronize()
                h.dev.record_stream(self.stream)
                h.dev = None

    def _h2d(self, h: _Handle):
        with torch.cuda.stream(self.stream):
            dev = torch.empty(h.shape, dtype=h.dtype, device=h.device)
            dev.copy_(h.host, non_blocking=True)
            h.h2d_event = torch.cuda.Event()
            h.h2d_event.record(self.stream)
        dev.record_stream(torch.cuda.current_stream())
        h.dev = dev

    def prefetch(self, layer: int):
        for h in self.layers.get(layer, []):
            if h.dev is None:
                self._h2d(h)

    def finish_layer_backward(self, layer: int):
        for h in self.layers.pop(layer, []):
            h.dev = None
            h.host = None
        if not self.layers:
            self.by_storage.clear()

    def reset(self):
        self.layers.clear()
        self.by_storage.clear()
        self.current_layer = -1


def install_swap_attention(model_chunks, args=None, swap_modules: Optional[str] = None, manager: Optional[SwapManager] = None):
    """Wrap every transformer layer (or the named sub-modules of it) so that tensors saved inside are swapped."""
    mgr = manager or SwapManager()
    names = (swap_modules or getattr(args, "swap_modules", None) or "input_layernorm,self_attention,pre_mlp_layernorm").split(",")
    names = [n.strip() for n in names if n.strip()]
    alias = {"input_norm": "input_layernorm", "post_attention_norm": "pre_mlp_layernorm"}
    names = [alias.get(n, n) for n in names]
    layer_input_only = bool(getattr(args, "swap_layer_input", False)) and not getattr(args, "swap_attention", False)
    idx = 0
    for chunk in model_chunks:
        inner = chunk.module if hasattr(chunk, "module") else chunk
        layers = list(inner.decoder.layers) if hasattr(inner, "decoder") else []
        for layer in layers:
            li = idx
            idx += 1
            targets = [layer] if layer_input_only else [getattr(layer, n) for n in names if hasattr(layer, n)]

            def pre(mod, inp, li=li):
                if mgr.current_layer != li:
                    if li > 0:
                        mgr.release_device_copies(li - 1)
                    mgr.current_layer = li

            layer.register_forward_pre_hook(pre)
            for tgt in targets:
                orig = tgt.forward

                def wrapped(*a, _orig=orig, **k):
                    if not torch.is_grad_enabled() or not mgr.enabled:
                        return _orig(*a, **k)
                    with torch.autograd.graph.saved_tensors_hooks(mgr.pack, mgr.unpack):
                        return _orig(*a, **k)

                tgt.forward = wrapped

            def bwd_pre(mod, gout, li=li):
                mgr.prefetch(li - 1)          # bring the previous layer back while this one runs backward

            def bwd_post(mod, gin, gout, li=li):
                mgr.finish_layer_backward(li)

            layer.register_full_backward_pre_hook(bwd_pre)
            layer.register_full_backward_hook(bwd_post)
    return mgr
