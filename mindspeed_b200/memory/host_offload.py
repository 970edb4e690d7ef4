"""Saved-for-backward tensors of one region parked in pinned host memory (no layer bookkeeping, no prefetch).

``with OffloadSaved():`` around a piece of forward: every CUDA tensor of at least ``min_bytes`` that autograd saves inside is
copied to a pinned host buffer with ``cudaMemcpyAsync`` on a side stream (ordered after its producer) and the device copy is
given back to the allocator once that copy has run; when backward asks for it, it is copied back on the consuming stream.
Used for buffers that are large, needed late in backward and cheap to fetch compared with what runs beside them - the
un-permute input of a MoE layer (``--moe-unperm2-mem-optim-swap``; reference: the swap of the second un-permute's input
in mindspeed/core/transformer/moe/moe_feature/fb_overlap and ``--moe-unperm2-mem-optim-swap``, mindspeed/features_manager/moe/
fb_overlap.py:72-73).  On CPU tensors the hooks pass everything through.
"""
from __future__ import annotations

import torch

MIN_BYTES = 1 << 20


class _Parked:
    __slots__ = ("host", "event", "device", "dtype", "shape")


class OffloadSaved:
    _streams = {}
    stats = {"tensors": 0, "bytes": 0}

    def __init__(self, min_bytes: int = MIN_BYTES):
        self.min_bytes = min_bytes
        self._hooks = None

    @classmethod
    def _side(cls, device):
        s = cls._streams.get(device)
        if s is None:
            s = cls._streams[device] = torch.cuda.Stream(device=device)
        return s

    def _pack(self, t: torch.Tensor):
        if (not t.is_cuda or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < self.min_bytes
                or not t.is_contiguous()):
            return t
        side = self._side(t.device)
        p = _Parked()
        p.device, p.dtype, p.shape = t.device, t.dtype, t.shape
        p.host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        side.wait_stream(torch.cuda.current_stream(t.device))
        t.record_stream(side)                          # the device memory may be reused only after the copy has run
        with torch.cuda.stream(side):
            p.host.copy_(t, non_blocking=True)
            p.event = side.record_event()
        OffloadSaved.stats["tensors"] += 1
        OffloadSaved.stats["bytes"] += t.numel() * t.element_size()
        return p

    @staticmethod
    def _unpack(obj):
        if not isinstance(obj, _Parked):
            return obj
        torch.cuda.current_stream(obj.device).wait_event(obj.event)
        dev = torch.empty(obj.shape, dtype=obj.dtype, device=obj.device)
        dev.copy_(obj.host, non_blocking=True)
        return dev

    def __enter__(self):
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        return self._hooks.__exit__(*exc)
