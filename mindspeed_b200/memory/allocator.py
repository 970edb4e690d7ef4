"""Python face of the native caching allocator (csrc/include/msb_caching_allocator.hpp).

  HostCachingAllocator   the allocator over a host-memory (optionally size-limited) backend - used by the CPU tests and
                         by the policy simulators, which replay allocation traces against it;
  install()              make the device build the allocator of this process' CUDA tensors
                         (torch.cuda.memory.CUDAPluggableAllocator; must run before the first CUDA allocation);
  device_stats / set_limit / set_tags / enable_trace / read_trace / set_pressure_callback
                         controls of the installed device allocator.

The pressure callback is what connects the allocator to the memory features: when a request cannot be served the
allocator calls back into Python before giving up, and the swap / adaptive-recompute managers release memory there
(reference: CheckAndSwapOutForOOM in mindspeed/ops/csrc/pluggable_allocator/smart_swap/NPUSwapManager.h:430 and the
memory-pressure hooks of adaptive_recomputing/NpuCachingCustomAllocator.cpp).
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, List, Optional

from ..utils.host_lib import host_lib


class Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("allocated_bytes", "reserved_bytes", "peak_allocated_bytes", "peak_reserved_bytes", "num_mallocs", "num_frees",
                 "num_segments", "num_segment_allocs", "num_pressure_events", "num_cache_flushes", "largest_free_block",
                 "free_bytes_in_cache")]

    def as_dict(self) -> Dict[str, int]:
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class TraceEvent(ctypes.Structure):
    _fields_ = [("seq", ctypes.c_uint64), ("addr", ctypes.c_uint64), ("size", ctypes.c_uint64), ("stream", ctypes.c_uint64),
                ("step", ctypes.c_int32), ("phase", ctypes.c_int32), ("is_free", ctypes.c_int32), ("pad", ctypes.c_int32)]


PRESSURE_CB = ctypes.CFUNCTYPE(ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p)


def _events(buf, n) -> List[Dict[str, int]]:
    return [dict(seq=int(e.seq), addr=int(e.addr), size=int(e.size), stream=int(e.stream), step=int(e.step),
                 phase=int(e.phase), is_free=bool(e.is_free)) for e in buf[:n]]


class HostCachingAllocator:
    def __init__(self, backend_capacity_bytes: int = 0):
        L = host_lib()
        L.msb_halloc_create.restype = ctypes.c_void_p
        L.msb_halloc_malloc.restype = ctypes.c_void_p
        L.msb_halloc_malloc.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_ulonglong]
        L.msb_halloc_free.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.msb_halloc_empty_cache.restype = ctypes.c_ulonglong
        L.msb_halloc_empty_cache.argtypes = [ctypes.c_void_p]
        L.msb_halloc_set_limit.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong]
        L.msb_halloc_set_tags.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        L.msb_halloc_set_pressure_callback.argtypes = [ctypes.c_void_p, PRESSURE_CB, ctypes.c_void_p]
        L.msb_halloc_enable_trace.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong]
        L.msb_halloc_read_trace.restype = ctypes.c_ulonglong
        L.msb_halloc_read_trace.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int]
        L.msb_halloc_stats.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.msb_halloc_block_size.restype = ctypes.c_ulonglong
        L.msb_halloc_block_size.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.msb_halloc_destroy.argtypes = [ctypes.c_void_p]
        L.msb_halloc_backend_in_use.restype = ctypes.c_ulonglong
        self.L = L
        self.h = L.msb_halloc_create(ctypes.c_ulonglong(backend_capacity_bytes))
        self._cb = None

    def malloc(self, nbytes: int, stream: int = 0) -> Optional[int]:
        return self.L.msb_halloc_malloc(self.h, nbytes, stream)

    def free(self, ptr: int) -> int:
        return self.L.msb_halloc_free(self.h, ptr)

    def empty_cache(self) -> int:
        return int(self.L.msb_halloc_empty_cache(self.h))

    def set_limit(self, nbytes: int):
        self.L.msb_halloc_set_limit(self.h, nbytes)

    def set_tags(self, step: int, phase: int):
        self.L.msb_halloc_set_tags(self.h, step, phase)

    def set_pressure_callback(self, fn: Optional[Callable[[int, int], int]]):
        """``fn(bytes_needed, device) -> bytes released``; it may call ``free`` on this allocator."""
        self._cb = PRESSURE_CB(lambda need, dev, _u: int(fn(int(need), int(dev)))) if fn is not None else PRESSURE_CB(0)
        self.L.msb_halloc_set_pressure_callback(self.h, self._cb, None)

    def enable_trace(self, capacity: int = 1 << 16):
        self.L.msb_halloc_enable_trace(self.h, capacity)

    def read_trace(self, clear: bool = True, max_events: int = 1 << 16):
        buf = (TraceEvent * max_events)()
        n = int(self.L.msb_halloc_read_trace(self.h, buf, max_events, int(clear)))
        return _events(buf, n)

    def stats(self) -> Dict[str, int]:
        s = Stats()
        self.L.msb_halloc_stats(self.h, ctypes.byref(s))
        return s.as_dict()

    def block_size(self, ptr: int) -> int:
        return int(self.L.msb_halloc_block_size(self.h, ptr))

    def backend_in_use(self) -> int:
        return int(self.L.msb_halloc_backend_in_use())

    def close(self):
        if self.h:
            self.L.msb_halloc_destroy(self.h)
            self.h = None


# ---- device allocator ------------------------------------------------------------------------------------------
_INSTALLED = {"done": False, "cb": None}


def install() -> bool:
    """Route this process' CUDA allocations through the native allocator.  Returns False when CUDA tensors already
    exist (torch only allows the switch before its own allocator has been used) or no GPU is present."""
    import torch
    from ..ops import loader
    if _INSTALLED["done"]:
        return True
    if not torch.cuda.is_available():
        return False
    loader.require_lib()
    try:
        alloc = torch.cuda.memory.CUDAPluggableAllocator(loader.LIB_PATH, "msb_torch_malloc", "msb_torch_free")
        torch.cuda.memory.change_current_allocator(alloc)
    except RuntimeError:
        return False
    _INSTALLED["done"] = True
    return True


def installed() -> bool:
    return _INSTALLED["done"]


def _dev(device):
    import torch
    return torch.cuda.current_device() if device is None else int(device)


def device_stats(device=None) -> Dict[str, int]:
    from ..ops import loader
    s = Stats()
    loader.require_lib().msb_dalloc_stats(_dev(device), ctypes.byref(s))
    return s.as_dict()


def set_limit(nbytes: int, device=None):
    from ..ops import loader
    loader.require_lib().msb_dalloc_set_limit(_dev(device), ctypes.c_ulonglong(nbytes))


def set_tags(step: int, phase: int, device=None):
    from ..ops import loader
    loader.require_lib().msb_dalloc_set_tags(_dev(device), step, phase)


def enable_trace(capacity: int = 1 << 18, device=None):
    from ..ops import loader
    loader.require_lib().msb_dalloc_enable_trace(_dev(device), ctypes.c_ulonglong(capacity))


def read_trace(clear: bool = True, max_events: int = 1 << 18, device=None):
    from ..ops import loader
    L = loader.require_lib()
    L.msb_dalloc_read_trace.restype = ctypes.c_ulonglong
    buf = (TraceEvent * max_events)()
    n = int(L.msb_dalloc_read_trace(_dev(device), buf, ctypes.c_ulonglong(max_events), int(clear)))
    return _events(buf, n)


def set_pressure_callback(fn: Optional[Callable[[int, int], int]], device=None):
    from ..ops import loader
    L = loader.require_lib()
    cb = PRESSURE_CB(lambda need, dev, _u: int(fn(int(need), int(dev)))) if fn is not None else PRESSURE_CB(0)
    _INSTALLED["cb"] = cb     # keep the trampoline alive
    L.msb_dalloc_set_pressure_callback.argtypes = [ctypes.c_int, PRESSURE_CB, ctypes.c_void_p]
    L.msb_dalloc_set_pressure_callback(_dev(device), cb, None)


def empty_cache(device=None) -> int:
    from ..ops import loader
    L = loader.require_lib()
    L.msb_dalloc_empty_cache.restype = ctypes.c_ulonglong
    return int(L.msb_dalloc_empty_cache(_dev(device)))
