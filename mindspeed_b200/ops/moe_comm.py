"""Host side of csrc/kernels/moe_comm.cu: MoE dispatch / combine over NVLink peer memory.

``RoutingPlan`` holds the index tables of one MoE layer call (all derived on the device from the all-gathered
per-expert token counts); ``dispatch`` and ``combine`` are autograd functions whose backward is each other's kernel.

Layout on the expert owner (rank d): rows sorted by [local expert][source rank][token order on the source] - the
layout the grouped GEMM consumes, so no regrouping pass follows the transfer.

Staging: every call copies its payload once into one of two slots of the symmetric heap (slot = call parity).  A
slot is rewritten two calls later; the call in between starts with a handshake that every rank passes only after
it has finished the earlier call, so the rewrite cannot race with a peer that is still reading.
reference: the fused dispatch / combine ops behind --moe-alltoall-mc2 and the all-to-all dispatcher contract in
mindspeed/core/transformer/moe/moe_feature/overlap/token_dispatcher.py:519-975.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from . import gemm as G
from . import loader
from ..parallel.symm_mem import SymmetricHeap, get_heap

MAX_RANKS = 8


class _MoeArgs(ctypes.Structure):
    _fields_ = [("out", ctypes.c_void_p), ("out_probs", ctypes.c_void_p),
                ("peer_rows", ctypes.c_void_p * 8), ("peer_tok", ctypes.c_void_p * 8), ("peer_probs", ctypes.c_void_p * 8),
                ("chunk_dst_start", ctypes.c_void_p), ("chunk_src_start", ctypes.c_void_p), ("map", ctypes.c_void_p),
                ("rank_in_expert", ctypes.c_void_p), ("dst_row_base", ctypes.c_void_p), ("R", ctypes.c_longlong),
                ("row_cap", ctypes.c_longlong),
                ("T", ctypes.c_int), ("E", ctypes.c_int), ("E_loc", ctypes.c_int), ("row_bytes", ctypes.c_int),
                ("world", ctypes.c_int), ("rank", ctypes.c_int), ("n_chunks", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("flag_local", ctypes.c_void_p), ("flag_peer", ctypes.c_void_p * 8), ("status", ctypes.c_void_p),
                ("wait_limit_ms", ctypes.c_int)]


class MoeCommContext:
    """Per expert-parallel group: heap, the two staging slots, the call counter."""

    def __init__(self, group, slot_bytes: int):
        self.group = group
        self.slot_bytes = ((slot_bytes + 1023) // 1024) * 1024
        heap_bytes = 2 * self.slot_bytes + (1 << 20)
        self.heap: SymmetricHeap = get_heap(group, heap_bytes, tag="moe")
        self.slot_off = [self.heap.alloc("moe_stage0", self.slot_bytes), self.heap.alloc("moe_stage1", self.slot_bytes)]
        self.calls = 0

    def next_slot(self) -> int:
        s = self.slot_off[self.calls & 1]
        self.calls += 1
        return s


_CTX = {}


def context(group, slot_bytes: int) -> MoeCommContext:
    c = _CTX.get(tuple(dist.get_process_group_ranks(group)))
    if c is None:
        c = MoeCommContext(group, slot_bytes)
        _CTX[tuple(dist.get_process_group_ranks(group))] = c
    elif c.slot_bytes < slot_bytes:
        raise RuntimeError(f"MoE staging slot of {c.slot_bytes} bytes is too small for {slot_bytes}; raise "
                           "MSB200_MOE_STAGE_FACTOR before the first MoE layer runs")
    return c


def reset():
    _CTX.clear()


def stage_factor() -> float:
    return float(os.environ.get("MSB200_MOE_STAGE_FACTOR", "2.0"))


class RoutingPlan:
    """Index tables of one dispatch/combine pair.  ``counts`` is the [ep, E] matrix of tokens that source rank s
    routes to global expert e (identical on every rank)."""

    def __init__(self, routing_map: torch.Tensor, counts: torch.Tensor, ep_rank: int, ep_size: int, n_routed: int,
                 n_recv: Optional[int] = None):
        T, E = routing_map.shape
        E_loc = E // ep_size
        dev = routing_map.device
        self.T, self.E, self.E_loc, self.ep, self.rank = T, E, E_loc, ep_size, ep_rank
        # ``n_recv`` (rows this rank receives) may be filled in later: everything else is computed on the device from
        # ``counts`` without a host read, so the tables and the staging copies can be queued before the one host sync
        self.n_routed, self.R = int(n_routed), (None if n_recv is None else int(n_recv))
        self.map_u8 = routing_map.to(torch.uint8).contiguous()
        self.rank_in_expert = (torch.cumsum(self.map_u8.to(torch.int32), dim=0, dtype=torch.int32) - 1).contiguous()
        # (expert, token) pairs of this rank in ascending (expert, token) order
        pairs = routing_map.t().contiguous().nonzero_static(size=self.n_routed)
        self.sorted_tok = pairs[:, 1].to(torch.int32).contiguous()
        self.sorted_flat = (pairs[:, 1] * E + pairs[:, 0]).contiguous()          # index into probs.view(-1)
        counts = counts.to(torch.int64)
        src_off = torch.cumsum(counts, dim=1) - counts                            # [ep, E] offset in the source's sorted list
        lo = ep_rank * E_loc
        mine = counts[:, lo:lo + E_loc]                                           # [ep, E_loc]
        sizes = mine.t().contiguous().view(-1)                                    # chunk order (local expert, source)
        self.chunk_dst_start = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), torch.cumsum(sizes, 0)]).contiguous()
        self.chunk_src_start = src_off[:, lo:lo + E_loc].t().contiguous().view(-1)
        per_e = counts.sum(0).view(ep_size, E_loc)
        first_row_of_expert = (torch.cumsum(per_e, dim=1) - per_e).view(-1)       # in the owner's layout
        self.dst_row_base = (first_row_of_expert + counts[:ep_rank].sum(0)).contiguous()


def build_plan_fused(routing_map: torch.Tensor, probs: torch.Tensor, counts_ld: torch.Tensor, ep_rank: int, ep_size: int,
                     n_routed: int) -> "RoutingPlan":
    """Same tables as ``RoutingPlan(...)`` from ONE kernel launch (csrc/kernels/moe_comm.cu: msb_moe_build_plan).
    ``counts_ld`` is the all-gathered [ep, ld] int64 matrix whose first E columns are the per-expert counts."""
    from ._dtypes import code
    L = loader.require_lib()
    T, E = routing_map.shape
    dev = routing_map.device
    plan = RoutingPlan.__new__(RoutingPlan)
    plan.T, plan.E, plan.E_loc, plan.ep, plan.rank = T, E, E // ep_size, ep_size, ep_rank
    plan.n_routed, plan.R = int(n_routed), None
    plan.map_u8 = routing_map.contiguous().view(torch.uint8) if routing_map.dtype == torch.bool else routing_map.to(torch.uint8).contiguous()
    plan.rank_in_expert = torch.empty(T, E, dtype=torch.int32, device=dev)
    cap = list_capacity(T, E)
    plan.sorted_tok = torch.empty(max(1, plan.n_routed), dtype=torch.int32, device=dev)
    plan.sorted_probs = torch.empty(max(1, plan.n_routed), dtype=torch.float32, device=dev)
    n_chunks = plan.E_loc * ep_size
    tables = torch.empty(2 * n_chunks + 1 + E, dtype=torch.int64, device=dev)
    plan.chunk_dst_start = tables[:n_chunks + 1]
    plan.chunk_src_start = tables[n_chunks + 1:2 * n_chunks + 1]
    plan.dst_row_base = tables[2 * n_chunks + 1:]
    plan.sorted_flat = None
    pc = probs.contiguous()
    if pc.dtype not in (torch.float32, torch.bfloat16):
        pc = pc.float()
    cl = counts_ld.contiguous()
    loader.check(L.msb_moe_build_plan(loader.p(plan.map_u8), loader.p(pc), code(pc.dtype), loader.p(cl), int(cl.shape[1]), T, E, plan.E_loc,
                                      ep_size, ep_rank, loader.p(plan.rank_in_expert), loader.p(plan.sorted_tok), loader.p(plan.sorted_probs),
                                      loader.p(plan.chunk_dst_start), loader.p(plan.chunk_src_start), loader.p(plan.dst_row_base),
                                      ctypes.c_longlong(min(cap, max(1, plan.n_routed))), ctypes.c_void_p(loader.stream_ptr())),
                 "moe_build_plan")
    plan._keep = (pc, cl)
    return plan


def _launch(fn_name: str, ctx: MoeCommContext, plan: RoutingPlan, out, out_probs, rows_off: int, tok_off: Optional[int],
            probs_off: Optional[int], row_bytes: int, row_cap: int = 1):
    L = loader.require_lib()
    h = ctx.heap
    a = _MoeArgs()
    a.out = out.data_ptr() if out.numel() else None
    a.out_probs = out_probs.data_ptr() if out_probs is not None else None
    for r in range(h.world):
        a.peer_rows[r] = h.ptr(r, rows_off)
        a.peer_tok[r] = h.ptr(r, tok_off) if tok_off is not None else None
        a.peer_probs[r] = h.ptr(r, probs_off) if probs_off is not None else None
        a.flag_peer[r] = h.ptr(r, 0)
    a.chunk_dst_start, a.chunk_src_start = plan.chunk_dst_start.data_ptr(), plan.chunk_src_start.data_ptr()
    a.map, a.rank_in_expert, a.dst_row_base = plan.map_u8.data_ptr(), plan.rank_in_expert.data_ptr(), plan.dst_row_base.data_ptr()
    a.R, a.T, a.E, a.E_loc, a.row_bytes, a.row_cap = plan.R, plan.T, plan.E, plan.E_loc, row_bytes, row_cap
    a.world, a.rank, a.n_chunks, a.epoch = h.world, h.rank, plan.E_loc * plan.ep, h.next_epoch()
    a.flag_local = h.ptr(h.rank, 0)
    a.status = G.status_word(out.device).data_ptr()
    a.wait_limit_ms = 0
    if a.out is None:
        a.out = h.ptr(h.rank, rows_off)     # never written: zero rows; keeps the launcher's null check simple
    loader.check(getattr(L, fn_name)(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), fn_name)


def _stage_dispatch(ctx: MoeCommContext, plan: RoutingPlan, x: torch.Tensor, sorted_probs: Optional[torch.Tensor]):
    """slot layout: [x: T*H] [token list: n_routed int32, padded] [probabilities: n_routed fp32]"""
    h = ctx.heap
    T, H = x.shape
    off = ctx.next_slot()
    tok_off = off + _up(T * H * x.element_size())
    probs_off = tok_off + _up(4 * list_capacity(T, plan.E))   # T and E are equal on every rank, so are the offsets
    if plan.n_routed > list_capacity(T, plan.E):
        raise RuntimeError("more routed (token, expert) pairs than the staging lists hold")
    h.tensor(off, (T, H), x.dtype).copy_(x)
    if plan.n_routed:
        h.tensor(tok_off, (plan.n_routed,), torch.int32).copy_(plan.sorted_tok)
        if sorted_probs is not None:
            h.tensor(probs_off, (plan.n_routed,), torch.float32).copy_(sorted_probs)
    return off, tok_off, (probs_off if sorted_probs is not None else None)


def list_capacity(T: int, E: int) -> int:
    """Entries of the token / probability lists behind the staged rows: up to 32 experts per token."""
    return T * min(E, 32)


def slot_bytes_needed(T: int, H: int, E: int, cap_rows: int, esize: int = 2) -> int:
    disp = _up(T * H * esize) + 2 * _up(4 * list_capacity(T, E))
    comb = _up(cap_rows * H * esize) + _up(4 * cap_rows)
    return max(disp, comb)


def _up(n, a=1024):
    return ((n + a - 1) // a) * a


def _stage_combine(ctx: MoeCommContext, plan: RoutingPlan, y: torch.Tensor, row_vals: Optional[torch.Tensor], cap_rows: int):
    """slot layout: [y: cap_rows * H] [per-row values: cap_rows fp32]"""
    h = ctx.heap
    R, H = y.shape
    off = ctx.next_slot()
    vals_off = off + _up(cap_rows * H * y.element_size())
    if R:
        h.tensor(off, (R, H), y.dtype).copy_(y)
        if row_vals is not None:
            h.tensor(vals_off, (R,), torch.float32).copy_(row_vals)
    return off, (vals_off if row_vals is not None else None)


def prestage_dispatch(comm: MoeCommContext, plan: RoutingPlan, x: torch.Tensor, probs: torch.Tensor):
    """Queue the staging copies of a dispatch (hidden states, sorted token list, sorted probabilities) ahead of the
    host synchronisation that determines the output size; returns the slot offsets for ``dispatch(..., staged=...)``."""
    with torch.no_grad():
        sorted_probs = plan.sorted_probs if getattr(plan, "sorted_probs", None) is not None \
            else probs.reshape(-1)[plan.sorted_flat].float()
        return _stage_dispatch(comm, plan, x.detach().contiguous(), sorted_probs)


class _Dispatch(torch.autograd.Function):
    """(x [T,H], probs [T,E]) -> (rows [R,H] in expert order, row probabilities [R])."""

    @staticmethod
    def forward(ctx, x, probs, comm: MoeCommContext, plan: RoutingPlan, cap_rows: int, staged=None):
        ctx.comm, ctx.plan, ctx.cap_rows = comm, plan, cap_rows
        ctx.x_dtype, ctx.p_dtype, ctx.H = x.dtype, probs.dtype, x.shape[1]
        if staged is not None:
            off, tok_off, probs_off = staged
        else:
            sorted_probs = plan.sorted_probs if getattr(plan, "sorted_probs", None) is not None \
                else probs.reshape(-1)[plan.sorted_flat].float()
            off, tok_off, probs_off = _stage_dispatch(comm, plan, x.contiguous(), sorted_probs)
        out = torch.empty(plan.R, x.shape[1], dtype=x.dtype, device=x.device)
        out_probs = torch.empty(plan.R, dtype=torch.float32, device=x.device)
        _launch("msb_moe_dispatch", comm, plan, out, out_probs, off, tok_off, probs_off, x.shape[1] * x.element_size())
        return out, out_probs.to(probs.dtype)

    @staticmethod
    def backward(ctx, d_rows, d_row_probs):
        comm, plan = ctx.comm, ctx.plan
        d_rows = d_rows.contiguous()
        vals = d_row_probs.float().contiguous() if d_row_probs is not None else None
        off, vals_off = _stage_combine(comm, plan, d_rows, vals, ctx.cap_rows)
        dx = torch.empty(plan.T, ctx.H, dtype=ctx.x_dtype, device=d_rows.device)
        dprobs = torch.zeros(plan.T, plan.E, dtype=torch.float32, device=d_rows.device) if vals is not None else None
        _launch("msb_moe_combine", comm, plan, dx, dprobs, off, None, vals_off, ctx.H * d_rows.element_size(),
                ctx.cap_rows)
        return dx, (dprobs.to(ctx.p_dtype) if dprobs is not None else None), None, None, None, None


class _Combine(torch.autograd.Function):
    """rows [R,H] (expert order, already weighted) -> [T,H]: sum of each token's expert outputs."""

    @staticmethod
    def forward(ctx, y, comm: MoeCommContext, plan: RoutingPlan, cap_rows: int):
        ctx.comm, ctx.plan = comm, plan
        y = y.contiguous()
        off, _ = _stage_combine(comm, plan, y, None, cap_rows)
        out = torch.empty(plan.T, y.shape[1], dtype=y.dtype, device=y.device)
        _launch("msb_moe_combine", comm, plan, out, None, off, None, None, y.shape[1] * y.element_size(), cap_rows)
        return out

    @staticmethod
    def backward(ctx, d_out):
        comm, plan = ctx.comm, ctx.plan
        d_out = d_out.contiguous()
        off, tok_off, _ = _stage_dispatch(comm, plan, d_out, None)
        dy = torch.empty(plan.R, d_out.shape[1], dtype=d_out.dtype, device=d_out.device)
        _launch("msb_moe_dispatch", comm, plan, dy, None, off, tok_off, None, d_out.shape[1] * d_out.element_size())
        return dy, None, None, None


def dispatch(x, probs, comm, plan, cap_rows, staged=None):
    return _Dispatch.apply(x, probs, comm, plan, cap_rows, staged)


def combine(y, comm, plan, cap_rows):
    return _Combine.apply(y, comm, plan, cap_rows)
