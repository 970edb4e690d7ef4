"""Deferred weight-gradient queue (dW / dX split).

Linear layers whose ``wgrad_deferral`` is set push ``(input, grad_output, weight)``
instead of running the weight-gradient GEMM; a pipeline schedule later calls
``pop()`` at a point where the GEMMs hide communication (pipeline p2p, MoE
all-to-all).  With sequence parallelism the stored input is the shard, and ``pop``
all-gathers the next entry's input on a side stream while the current entry's GEMM
runs (reference: mindspeed/core/weight_grad_store.py:63-240 and
mindspeed/core/transformer/moe/moe_feature/fb_overlap/modules/weight_grad_store.py:35-171).
"""
from __future__ import annotations

import queue
from typing import List

import torch


class WeightGradStore:
    _enabled = False
    _cache: List[tuple] = []
    _queue: "queue.Queue[List[tuple]]" = queue.Queue()
    _gather_stream = None
    swap_to_host = False           # park the stored inputs / output gradients in pinned host memory between flush and pop
    _offload = None
    _fresh = None                  # swap mode: the most recently flushed micro-batch, still on the device

    @classmethod
    def _park(cls, entries):
        if not cls.swap_to_host:
            return entries
        if cls._offload is None:
            from ..memory.host_offload import OffloadSaved
            cls._offload = OffloadSaved(min_bytes=1 << 16)
        pk = cls._offload._pack
        return [(pk(x), pk(dy), w, sp, g, f) for x, dy, w, sp, g, f in entries]

    @classmethod
    def _fetch(cls, entries):
        if cls._offload is None:
            return entries
        up = cls._offload._unpack
        return [(up(x), up(dy), w, sp, g, f) for x, dy, w, sp, g, f in entries]

    @classmethod
    def enable(cls, flag: bool = True):
        cls._enabled = flag

    @classmethod
    def enabled(cls) -> bool:
        return cls._enabled

    @classmethod
    def put(cls, x, dy, weight, sequence_parallel, group, fusion):
        cls._cache.append((x, dy, weight, sequence_parallel, group, fusion))

    @classmethod
    def flush(cls):
        """Close the current micro-batch: everything put since the last flush pops together."""
        if cls.swap_to_host:
            # the newest micro-batch stays on the device: if its W comes next it is popped as it is; it is parked only when
            # another backward arrives first, i.e. when its W has been deferred
            if cls._fresh is not None:
                cls._queue.put(cls._park(cls._fresh))
            cls._fresh = cls._cache
        else:
            cls._queue.put(cls._cache)
        cls._cache = []

    @classmethod
    def is_empty(cls) -> bool:
        return cls._queue.empty() and cls._fresh is None

    @classmethod
    def clear(cls):
        cls._cache = []
        cls._fresh = None
        cls._queue = queue.Queue()

    @classmethod
    def _gather(cls, entry):
        from . import mappings as M
        x, dy, weight, sp, group, fusion = entry
        if not sp:
            return x, None
        if torch.cuda.is_available() and x.is_cuda:
            if cls._gather_stream is None:
                cls._gather_stream = torch.cuda.Stream()
            cls._gather_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cls._gather_stream):
                total, h = M.all_gather_first_dim(x, group, async_op=True)
            return total, h
        return M.all_gather_first_dim(x, group), None

    @classmethod
    @torch.no_grad()
    def pop(cls, num: int = -1) -> int:
        """Run the weight-gradient GEMMs of one flushed micro-batch (or ``num`` entries of it)."""
        from .comm_ops import get_ops
        from .layers import _wgrad
        if cls._fresh is not None:
            entries, cls._fresh = cls._fresh, None
        else:
            if cls._queue.empty():
                if not cls._cache:
                    return 0
                cls.flush()
                return cls.pop(num)
            entries = cls._fetch(cls._queue.get())
        if 0 <= num < len(entries):
            rest = entries[num:]
            entries = entries[:num]
            # put the remainder back at the front
            q2 = queue.Queue()
            q2.put(rest)
            while not cls._queue.empty():
                q2.put(cls._queue.get())
            cls._queue = q2
        ops = get_ops()
        nxt = cls._gather(entries[0]) if entries else None
        for i, e in enumerate(entries):
            total, h = nxt
            if i + 1 < len(entries):
                nxt = cls._gather(entries[i + 1])
            if h is not None:
                h.wait()
                if cls._gather_stream is not None:
                    torch.cuda.current_stream().wait_stream(cls._gather_stream)
            x, dy, weight, sp, group, fusion = e
            dw = _wgrad(ops, dy, total, weight, fusion)
            if dw is not None:
                # autograd is not involved here, so the data-parallel hook will not fire: add to the buffer directly
                if hasattr(weight, "main_grad"):
                    weight.main_grad.add_(dw.to(weight.main_grad.dtype))
                    cb = getattr(weight, "_main_grad_ready_cb", None)
                    if cb is not None:
                        cb(weight)
                else:
                    weight.grad = dw if weight.grad is None else weight.grad + dw
        return len(entries)

    @classmethod
    def pop_all(cls):
        n = 0
        while not cls._queue.empty() or cls._cache or cls._fresh is not None:
            n += cls.pop()
        return n
