"""Ulysses all-to-alls with the layout transform fused in (host side of csrc/kernels/a2a_strided.cu).

  seq_to_heads_fused(x [s/p, b, n, d])  -> [s, b, n/p, d]
  heads_to_seq_fused(x [s, b, n/p, d])  -> [s/p, b, n, d]

Each call stages its input once in one of two slots of a symmetric heap over the context-parallel group and launches
one pull kernel; the permute / contiguous passes of the library path disappear.  The two functions are each other's
backward.  Any dtype (the kernel copies bytes); rows (n/p * d elements) must be a multiple of 16 bytes.
reference: mindspeed/core/context_parallel/ulysses_context_parallel/ulysses_context_parallel.py:83-108.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import gemm as G
from . import loader
from ..parallel.symm_mem import SymmetricHeap, get_heap


class _Args(ctypes.Structure):
    _fields_ = [("peer", ctypes.c_void_p * 8), ("out", ctypes.c_void_p), ("rows", ctypes.c_longlong), ("src_base", ctypes.c_longlong),
                ("src_row_stride", ctypes.c_longlong), ("dst_src_stride", ctypes.c_longlong), ("dst_row_stride", ctypes.c_longlong),
                ("row_bytes", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("flag_local", ctypes.c_void_p), ("flag_peer", ctypes.c_void_p * 8), ("status", ctypes.c_void_p),
                ("wait_limit_ms", ctypes.c_int)]


class _Ctx:
    def __init__(self, group, slot_bytes):
        self.slot_bytes = ((slot_bytes + 1023) // 1024) * 1024
        self.heap: SymmetricHeap = get_heap(group, 2 * self.slot_bytes + (1 << 20), tag="ulysses")
        self.slots = [self.heap.alloc("a2a_stage0", self.slot_bytes), self.heap.alloc("a2a_stage1", self.slot_bytes)]
        self.calls = 0


_CTX = {}


def _ctx(group, nbytes) -> _Ctx:
    c = _CTX.get(tuple(dist.get_process_group_ranks(group)))
    if c is None:
        floor = int(os.environ.get("MSB200_ULYSSES_SLOT_MIB", "64")) << 20
        c = _Ctx(group, max(nbytes, floor))
        _CTX[tuple(dist.get_process_group_ranks(group))] = c
    if c.slot_bytes < nbytes:
        raise RuntimeError(f"Ulysses staging slot of {c.slot_bytes} bytes is too small for {nbytes}; raise MSB200_ULYSSES_SLOT_MIB")
    return c


def reset():
    _CTX.clear()


def eligible(x, group) -> bool:
    if group is None or not x.is_cuda or loader.lib() is None:
        return False
    p = dist.get_world_size(group)
    return 2 <= p <= 8


def _pull(x, group, out_shape, rows, src_base, src_row_stride, dst_src_stride, dst_row_stride, row_bytes):
    L = loader.require_lib()
    xc = x.contiguous()
    nbytes = xc.numel() * xc.element_size()
    c = _ctx(group, nbytes)
    h = c.heap
    off = c.slots[c.calls & 1]
    c.calls += 1
    h.tensor(off, (xc.numel(),), xc.dtype).copy_(xc.reshape(-1))
    out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    a = _Args()
    for r in range(h.world):
        a.peer[r] = h.ptr(r, off)
        a.flag_peer[r] = h.ptr(r, 0)
    a.out = out.data_ptr()
    a.rows, a.src_base, a.src_row_stride = rows, src_base, src_row_stride
    a.dst_src_stride, a.dst_row_stride, a.row_bytes = dst_src_stride, dst_row_stride, row_bytes
    a.world, a.rank, a.epoch = h.world, h.rank, h.next_epoch()
    a.flag_local = h.ptr(h.rank, 0)
    a.status = G.status_word(x.device).data_ptr()
    a.wait_limit_ms = 0
    loader.check(L.msb_a2a_strided_pull(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "a2a_strided_pull")
    return out


def _s2h(x, group):
    p, me = dist.get_world_size(group), dist.get_rank(group)
    sl, b, n, d = x.shape
    nl = n // p
    es = x.element_size()
    row = nl * d * es
    if n % p != 0 or row % 16 != 0:
        raise ValueError("heads must divide by the group size and a head slice must be a multiple of 16 bytes")
    return _pull(x, group, (p * sl, b, nl, d), rows=sl * b, src_base=me * row, src_row_stride=n * d * es,
                 dst_src_stride=sl * b * row, dst_row_stride=row, row_bytes=row)


def _h2s(x, group):
    p, me = dist.get_world_size(group), dist.get_rank(group)
    s, b, nl, d = x.shape
    sl = s // p
    es = x.element_size()
    row = nl * d * es
    if s % p != 0 or row % 16 != 0:
        raise ValueError("sequence must divide by the group size and a head slice must be a multiple of 16 bytes")
    return _pull(x, group, (sl, b, p * nl, d), rows=sl * b, src_base=me * sl * b * row, src_row_stride=row,
                 dst_src_stride=row, dst_row_stride=p * row, row_bytes=row)


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _s2h(x, group)

    @staticmethod
    def backward(ctx, g):
        return _h2s(g, ctx.group), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _h2s(x, group)

    @staticmethod
    def backward(ctx, g):
        return _s2h(g, ctx.group), None


def seq_to_heads_fused(x, group):
    return _SeqToHeads.apply(x, group)


def heads_to_seq_fused(x, group):
    return _HeadsToSeq.apply(x, group)
