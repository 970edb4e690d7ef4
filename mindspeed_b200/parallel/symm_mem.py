"""Symmetric device memory over a process group (host side of csrc/runtime/symm.cu).

Every rank of the group allocates one equally sized heap; IPC handles are exchanged over the group and every rank
maps all peers.  The first 8 KiB of a heap hold synchronisation words (entry flags, exit flags, arrival counter,
per-tile ready counters); named buffers are carved from the rest.  Kernels receive the table of peer base pointers.

This is the B200 replacement for the communicator handles the reference passes into its fused vendor kernels
(mindspeed/core/tensor_parallel/mc2_feature/linear_function.py:7-20, mindspeed/ops/lcal_functional.py:31-84).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..ops import loader

FLAG_BYTES = 8192
MAX_RANKS = 8
READY_OFFSET_WORDS = 64  # ready counters start here (u32 index)


class _RawCuda:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricHeap:
    def __init__(self, group, nbytes: int):
        L = loader.require_lib()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_RANKS:
            raise RuntimeError(f"symmetric heaps support at most {MAX_RANKS} ranks (one NVSwitch domain)")
        self.nbytes = FLAG_BYTES + ((nbytes + 1023) // 1024) * 1024
        p = ctypes.c_void_p()
        loader.check(L.msb_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(p)), "symm_alloc")
        self.local_ptr = p.value
        hb = (ctypes.c_ubyte * 64)()
        loader.check(L.msb_symm_export(ctypes.c_void_p(self.local_ptr), hb), "symm_export")
        handles: List[bytes] = [None] * self.world
        dist.all_gather_object(handles, bytes(hb), group=group)
        self.peer_ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
            else:
                q = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                loader.check(L.msb_symm_import(buf, ctypes.byref(q)), "symm_import")
                self.peer_ptrs.append(q.value)
        self._raw = torch.as_tensor(_RawCuda(self.local_ptr, self.nbytes), device=torch.device("cuda", torch.cuda.current_device()))
        self._cursor = FLAG_BYTES
        self._named: Dict[str, Tuple[int, int]] = {}
        self.epoch = 0
        dist.barrier(group=group)

    # ---- layout ----
    def alloc(self, name: str, nbytes: int) -> int:
        """Offset of a named buffer (allocated once; same offset on every rank because calls are SPMD)."""
        if name in self._named:
            off, size = self._named[name]
            if size >= nbytes:
                return off
            raise RuntimeError(f"symmetric buffer '{name}' of {size} bytes is too small for {nbytes}")
        off = self._cursor
        size = ((nbytes + 1023) // 1024) * 1024
        if off + size > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted: need {size} more bytes at {off} of {self.nbytes}")
        self._cursor += size
        self._named[name] = (off, size)
        return off

    def tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self._raw[offset:offset + nb].view(dtype).view(*shape)

    def ptr(self, rank: int, offset: int = 0) -> int:
        return self.peer_ptrs[rank] + offset

    def ptr_table(self, offset: int = 0):
        arr = (ctypes.c_void_p * MAX_RANKS)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r] + offset
        return arr

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def close(self):
        L = loader.lib()
        if L is None or self.local_ptr is None:
            return
        torch.cuda.synchronize()
        for r, q in enumerate(self.peer_ptrs):
            if r != self.rank:
                L.msb_symm_close(ctypes.c_void_p(q))
        L.msb_symm_free(ctypes.c_void_p(self.local_ptr))
        self.local_ptr = None


_HEAPS: Dict[int, SymmetricHeap] = {}


def get_heap(group, nbytes: int, tag: str = "tp") -> SymmetricHeap:
    """One heap per (group, tag): kernel families with their own flag words and buffers keep separate heaps."""
    # keyed by the group's global ranks, not by object identity: a destroyed and re-created group must not pick up a stale heap
    key = (tuple(dist.get_process_group_ranks(group)) if group is not None else ("world",), tag)
    h = _HEAPS.get(key)
    if h is None:
        h = SymmetricHeap(group, nbytes)
        _HEAPS[key] = h
    return h


def destroy_heaps():
    for h in _HEAPS.values():
        h.close()
    _HEAPS.clear()
