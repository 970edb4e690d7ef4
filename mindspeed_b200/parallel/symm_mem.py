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


GUARD_BYTES = 1024
GUARD_PATTERN = 0xA5


class HeapLayout:
    """Offsets of named buffers inside a heap of ``nbytes`` (the first ``FLAG_BYTES`` are the synchronisation words).
    With ``guard`` > 0 every buffer is followed by ``guard`` canary bytes that no kernel may touch: ``fill_guards`` writes
    the pattern, ``check_guards`` names the buffers whose canary has been overwritten (a write past the buffer's end by a
    local kernel or by a peer's store).  The sizes and offsets are the same on every rank because allocation calls are SPMD."""

    def __init__(self, nbytes: int, guard: int = 0):
        self.nbytes, self.guard = nbytes, guard
        self.cursor = FLAG_BYTES
        self.named: Dict[str, Tuple[int, int]] = {}

    def alloc(self, name: str, nbytes: int) -> Tuple[int, bool]:
        """(offset, newly allocated)."""
        if name in self.named:
            off, size = self.named[name]
            if size >= nbytes:
                return off, False
            raise RuntimeError(f"symmetric buffer '{name}' of {size} bytes is too small for {nbytes}")
        off = self.cursor
        size = ((nbytes + 1023) // 1024) * 1024
        if off + size + self.guard > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted: need {size + self.guard} more bytes at {off} of {self.nbytes}")
        self.cursor += size + self.guard
        self.named[name] = (off, size)
        return off, True

    def guard_range(self, name: str) -> Tuple[int, int]:
        off, size = self.named[name]
        return off + size, off + size + self.guard

    def fill_guard(self, raw: torch.Tensor, name: str):
        if self.guard:
            a, b = self.guard_range(name)
            raw[a:b].fill_(GUARD_PATTERN)

    def check_guards(self, raw: torch.Tensor) -> List[str]:
        """Names of the buffers whose canary no longer holds the pattern (one device-to-host read per buffer)."""
        bad = []
        if self.guard:
            for name in self.named:
                a, b = self.guard_range(name)
                if bool((raw[a:b] != GUARD_PATTERN).any()):
                    bad.append(name)
        return bad


def canaries_enabled() -> bool:
    import os
    return os.environ.get("MSB200_HEAP_CANARIES", "0") == "1"


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
        # MSB200_HEAP_CANARIES=1 (debugging): guard bytes behind every buffer, verified by check_canaries(); the heap itself is
        # not enlarged, so a configuration that fills it exactly needs a larger heap in this mode
        self.layout = HeapLayout(self.nbytes, GUARD_BYTES if canaries_enabled() else 0)
        self.epoch = 0
        dist.barrier(group=group)

    # ---- layout ----
    def alloc(self, name: str, nbytes: int) -> int:
        """Offset of a named buffer (allocated once; same offset on every rank because calls are SPMD)."""
        off, new = self.layout.alloc(name, nbytes)
        if new:
            self.layout.fill_guard(self._raw, name)
        return off

    def check_canaries(self):
        """Debug mode only: raise if a kernel (of this rank or a peer) wrote past the end of a named buffer."""
        if not self.layout.guard:
            return
        torch.cuda.synchronize()
        bad = self.layout.check_guards(self._raw)
        if bad:
            raise RuntimeError(f"symmetric heap of rank {self.rank}: guard bytes overwritten behind {bad}")

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


def check_all_canaries():
    """Debug mode (``MSB200_HEAP_CANARIES=1``): verify the guard bytes of every heap; called by the training loop after a step."""
    for h in _HEAPS.values():
        h.check_canaries()


def destroy_heaps():
    for h in _HEAPS.values():
        h.close()
    _HEAPS.clear()
