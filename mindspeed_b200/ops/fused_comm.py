"""Fused GEMM + collective back end (optimisation level 2): drives csrc/kernels/gemm_sm100.cu in its
all-gather and reduce-scatter modes over a symmetric heap.

  allgather_matmul:      y = allgather(x) @ W^T  (or @ W)   one kernel: peer pulls + tcgen05 tiles
  matmul_reduce_scatter: y = reduce_scatter(x @ W^T)        one kernel (tiles + pushes) + the owner-side reduction

Both are numerically interchangeable with the library path within bf16 rounding: partial sums cross NVLink in bf16
and are added in fp32 in a fixed rank order, so results are run-to-run deterministic.
reference semantics: npu_all_gather_base_mm / npu_mm_reduce_scatter_base as used by
mindspeed/core/tensor_parallel/mc2_feature/linear_function.py:23-246.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import loader
from . import gemm as G
from ..parallel.comm_ops import Sm100Ops
from ..parallel.symm_mem import READY_OFFSET_WORDS, SymmetricHeap, get_heap

MAX_SRC = 8


class _CommArgs(ctypes.Structure):
    _fields_ = [("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("D", ctypes.c_void_p),
                ("peer_buf", ctypes.c_void_p * MAX_SRC), ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("b_mn_major", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("flag_local", ctypes.c_void_p), ("flag_peer", ctypes.c_void_p * MAX_SRC), ("ready", ctypes.c_void_p),
                ("status", ctypes.c_void_p)]


def _heap_bytes(default_mib=640):
    return int(os.environ.get("MSB200_SYMM_HEAP_MIB", default_mib)) * 1024 * 1024


def _buf_bytes(request):
    """Named buffers are sized once; reserve a floor so later, somewhat larger shapes still fit."""
    return max(request, int(os.environ.get("MSB200_SYMM_BUF_MIB", 128)) * 1024 * 1024)


class _Comm2Args(ctypes.Structure):
    """Arguments of the CTA-pair fused kernels (csrc/kernels/gemm2_comm_sm100.cu, struct MsbComm2Args)."""
    _fields_ = [("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("D", ctypes.c_void_p),
                ("peer_buf", ctypes.c_void_p * MAX_SRC), ("residual", ctypes.c_void_p), ("ar_out", ctypes.c_void_p * MAX_SRC),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("b_mn_major", ctypes.c_int),
                ("world", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("flag_local", ctypes.c_void_p), ("flag_peer", ctypes.c_void_p * MAX_SRC), ("status", ctypes.c_void_p),
                ("wait_limit_ms", ctypes.c_int), ("max_ctas", ctypes.c_int), ("timeline", ctypes.c_void_p)]


MODE_AG, MODE_RS = 1, 2
# 0: CTA-pair kernels wherever they cover the shape (default); 1: always the one-CTA fused kernels (comparisons)
_FORCE_ONE_CTA = os.environ.get("MSB200_FUSED_ONE_CTA", "0") != "0"
WAIT_LIMIT_MS = int(os.environ.get("MSB200_COMM_WAIT_MS", "10000"))


TIMELINE = None      # set to a uint64 [8] device tensor to collect CTA 0's time stamps of the next pair-kernel launch


def _pair_ok(L, m, n, k, ws, mode) -> bool:
    return (not _FORCE_ONE_CTA) and bool(L.msb_gemm2_comm_supported(m, n, k, ws, mode))


class _Ctx:
    """Per-process-group state: heap, buffer offsets, call parity."""

    def __init__(self, group):
        self.heap: SymmetricHeap = get_heap(group, _heap_bytes())
        self.ag_calls = 0

    def fill_pair(self, a: _Comm2Args, epoch: int, dev):
        h = self.heap
        a.world, a.rank, a.epoch = h.world, h.rank, epoch
        a.flag_local = h.ptr(h.rank, 0)
        for r in range(h.world):
            a.flag_peer[r] = h.ptr(r, 0)
        a.status = G.status_word(dev).data_ptr()
        a.wait_limit_ms = WAIT_LIMIT_MS
        a.max_ctas = 0
        a.timeline = TIMELINE.data_ptr() if TIMELINE is not None else None

    def fill_common(self, a: _CommArgs, epoch: int, dev):
        h = self.heap
        a.world, a.rank, a.epoch = h.world, h.rank, epoch
        a.flag_local = h.ptr(h.rank, 0)
        for r in range(h.world):
            a.flag_peer[r] = h.ptr(r, 0)
        a.ready = h.ptr(h.rank, 4 * READY_OFFSET_WORDS)
        a.status = G.status_word(dev).data_ptr()


_CTX = {}


def _ctx(group) -> _Ctx:
    key = tuple(dist.get_process_group_ranks(group))      # global ranks: survives re-creation of the group object
    c = _CTX.get(key)
    if c is None:
        c = _Ctx(group)
        _CTX[key] = c
    return c


def reset():
    _CTX.clear()


class FusedOps(Sm100Ops):
    name = "fused"
    gathered_is_view = True   # the gathered input returned by allgather_matmul lives in a recycled symmetric buffer
    # backward of a column-parallel linear: the weight-gradient GEMM (pure compute) runs on a side stream on
    # ``wgrad_ctas`` SMs while the GEMM->reduce-scatter kernel (mostly waiting on NVLink) runs on the remaining ones
    concurrent_wgrad = os.environ.get("MSB200_CONCURRENT_WGRAD", "0") != "0"   # opt-in: pays only when the dgrad kernel is NVLink-bound
    wgrad_ctas = int(os.environ.get("MSB200_WGRAD_CTAS", "96"))
    _side_stream = None

    @classmethod
    def dgrad_reduce_scatter_with_wgrad(cls, dy, w, total, main_grad, group):
        """dx = reduce_scatter(dy @ w) and main_grad += dy^T @ total, issued so that the two overlap on the GPU."""
        if cls._side_stream is None:
            cls._side_stream = torch.cuda.Stream()
        side, cur = cls._side_stream, torch.cuda.current_stream()
        n_sm = torch.cuda.get_device_properties(dy.device).multi_processor_count
        k = max(8, min(cls.wgrad_ctas, n_sm - 16))
        side.wait_stream(cur)
        with torch.cuda.stream(side), G.cta_limit(k):
            cls.wgrad(dy, total, main_grad)
        dy.record_stream(side)
        total.record_stream(side)
        with G.cta_limit(n_sm - k):
            dx = cls.matmul_reduce_scatter(dy, w, group, nt=False)
        cur.wait_stream(side)
        return dx

    @staticmethod
    def _eligible(x, w, group, rows_total, n_out, k):
        if group is None or not x.is_cuda or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return False
        ws = dist.get_world_size(group)
        return 2 <= ws <= MAX_SRC and rows_total % (ws * 128) == 0 and n_out % 8 == 0 and k % 8 == 0 and w.is_contiguous()

    @classmethod
    def allgather_matmul(cls, x, w, group, nt=True, need_gathered=False):
        ws = dist.get_world_size(group) if group is not None else 1
        x2 = x.reshape(-1, x.shape[-1])
        rows, k = x2.shape
        m = rows * ws
        n = w.shape[0] if nt else w.shape[1]
        if not cls._eligible(x, w, group, m, n, k):
            return Sm100Ops.allgather_matmul(x, w, group, nt, need_gathered)
        L = loader.require_lib()
        c = _ctx(group)
        h = c.heap
        parity = c.ag_calls & 1
        c.ag_calls += 1
        off = h.alloc(f"ag{parity}", _buf_bytes(m * k * 2))
        gathered = h.tensor(off, (m, k), torch.bfloat16)
        gathered[h.rank * rows:(h.rank + 1) * rows].copy_(x2)
        lead = (x.shape[0] * ws,) + tuple(x.shape[1:-1])
        y = torch.empty(*lead, n, dtype=torch.bfloat16, device=x.device)   # final shape: custom Functions must not return views
        pair = _pair_ok(L, m, n, k, ws, MODE_AG)
        a = _Comm2Args() if pair else _CommArgs()
        a.A, a.B, a.D = h.ptr(h.rank, off), w.data_ptr(), y.data_ptr()
        for r in range(ws):
            a.peer_buf[r] = h.ptr(r, off)
        a.M, a.N, a.K, a.b_mn_major = m, n, k, 0 if nt else 1
        if pair:
            c.fill_pair(a, h.next_epoch(), x.device)
            loader.check(L.msb_gemm2_allgather(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "gemm2_allgather")
        else:
            c.fill_common(a, h.next_epoch(), x.device)
            loader.check(L.msb_gemm_allgather(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "gemm_allgather")
        total = gathered.view(*lead, k) if need_gathered else None
        return y, total

    @classmethod
    def matmul_all_reduce(cls, x, w, group, nt=True):
        """y = all_reduce(x @ W): the fused GEMM -> reduce-scatter kernel followed by an all-gather of the reduced row
        shards (non-sequence-parallel tensor parallelism; reference: npu_mm_all_reduce_base / LCAL matmul_all_reduce)."""
        ws = dist.get_world_size(group) if group is not None else 1
        x2 = x.reshape(-1, x.shape[-1])
        n = w.shape[0] if nt else w.shape[1]
        if ws < 2 or not cls._eligible(x, w, group, x2.shape[0], n, x2.shape[1]):
            return Sm100Ops.matmul_all_reduce(x, w, group, nt)
        if _pair_ok(loader.require_lib(), x2.shape[0], n, x2.shape[1], ws, MODE_RS) and x2.is_contiguous() and x2.data_ptr() % 16 == 0:
            # one kernel: tiles -> owners' staging -> fp32 sum -> reduced rows written into every rank's output
            full = cls._pair_reduce_scatter(_ctx(group), x, x2, w, x2.shape[0], n, x2.shape[1], nt, None, all_reduce=True)
            return full.view(*x.shape[:-1], n)
        part = cls.matmul_reduce_scatter(x2, w, group, nt)
        full = torch.empty(x2.shape[0], n, dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(full, part.contiguous(), group=group)
        return full.view(*x.shape[:-1], n)

    @classmethod
    def matmul_all_reduce_add_rmsnorm(cls, x, w, residual, gamma, eps, group, nt=True):
        """(h, y) with h = all_reduce(x @ W) + residual and y = rmsnorm(h) * gamma.  The residual is added inside the
        owner-side reduction of the reduce-scatter, the norm runs on the row shard each rank owns (rows are
        independent), and one all-gather returns both results (reference: aclnnMatmulAllReduceAddRmsNorm)."""
        from .norm import rms_norm
        ws = dist.get_world_size(group) if group is not None else 1
        x2 = x.reshape(-1, x.shape[-1])
        n = w.shape[0] if nt else w.shape[1]
        res2 = residual.reshape(-1, n)
        if ws < 2 or not cls._eligible(x, w, group, x2.shape[0], n, x2.shape[1]):
            h = Sm100Ops.matmul_all_reduce(x, w, group, nt) + residual
            return h, rms_norm(h, gamma, eps)
        rows = x2.shape[0] // ws
        r = dist.get_rank(group)
        h_part = cls.matmul_reduce_scatter(x2, w, group, nt, residual=res2[r * rows:(r + 1) * rows].contiguous())
        y_part = rms_norm(h_part, gamma, eps)
        both = torch.stack([h_part, y_part]).contiguous()                      # [2, rows, n]
        out = torch.empty(ws, 2, rows, n, dtype=both.dtype, device=both.device)
        dist.all_gather_into_tensor(out, both, group=group)
        h = out[:, 0].reshape(*x.shape[:-1], n)
        y = out[:, 1].reshape(*x.shape[:-1], n)
        return h, y

    @classmethod
    def _pair_reduce_scatter(cls, c, x, x2, w, m, n, k, nt, residual, all_reduce):
        """GEMM -> reduce-scatter (-> all-gather) on the CTA-pair kernel: tiles go from the epilogue straight into the
        owners' staging slabs, the tail of the same kernel sums the slabs (+ residual).  With ``all_reduce`` the reduced
        rows are also written into every rank's copy of a symmetric [m, n] buffer, which is returned as a fresh tensor."""
        L = loader.require_lib()
        h = c.heap
        ws, rows = h.world, m // h.world
        off_stage = h.alloc("rs_stage", _buf_bytes(m * n * 2))
        a = _Comm2Args()
        a.A, a.B = x2.data_ptr(), w.data_ptr()
        for r in range(ws):
            a.peer_buf[r] = h.ptr(r, off_stage)
        a.M, a.N, a.K, a.b_mn_major = m, n, k, 0 if nt else 1
        a.residual = residual.data_ptr() if residual is not None else None
        out = None
        if all_reduce:
            off_ar = h.alloc("ar_out", _buf_bytes(m * n * 2))
            for r in range(ws):
                a.ar_out[r] = h.ptr(r, off_ar)
            a.D = None
        else:
            lead = (x.shape[0] // ws,) + tuple(x.shape[1:-1])
            out = torch.empty(*lead, n, dtype=torch.bfloat16, device=x.device)
            a.D = out.data_ptr()
        c.fill_pair(a, h.next_epoch(), x.device)
        loader.check(L.msb_gemm2_reduce_scatter(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "gemm2_reduce_scatter")
        if all_reduce:
            return h.tensor(off_ar, (m, n), torch.bfloat16).clone()     # the symmetric buffer is recycled by the next call
        return out

    @classmethod
    def matmul_reduce_scatter(cls, x, w, group, nt=True, residual=None):
        ws = dist.get_world_size(group) if group is not None else 1
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m, k = x2.shape
        n = w.shape[0] if nt else w.shape[1]
        if not cls._eligible(x, w, group, m, n, k) or x2.data_ptr() % 16 != 0:
            out = Sm100Ops.matmul_reduce_scatter(x, w, group, nt)
            return out if residual is None else out + residual.view_as(out)
        L = loader.require_lib()
        c = _ctx(group)
        h = c.heap
        rows = m // ws
        if residual is not None and (residual.dtype != torch.bfloat16 or not residual.is_contiguous() or residual.numel() != rows * n):
            raise ValueError("residual must be a contiguous bf16 tensor shaped like this rank's output shard")
        if _pair_ok(L, m, n, k, ws, MODE_RS):
            return cls._pair_reduce_scatter(c, x, x2, w, m, n, k, nt, residual, all_reduce=False)
        off_partial = h.alloc("rs_partial", _buf_bytes(m * n * 2))
        off_stage = h.alloc("rs_stage", _buf_bytes(m * n * 2))
        a = _CommArgs()
        a.A, a.B, a.D = x2.data_ptr(), w.data_ptr(), h.ptr(h.rank, off_partial)
        for r in range(ws):
            a.peer_buf[r] = h.ptr(r, off_stage)
        a.M, a.N, a.K, a.b_mn_major = m, n, k, 0 if nt else 1
        epoch = h.next_epoch()
        c.fill_common(a, epoch, x.device)
        st = ctypes.c_void_p(loader.stream_ptr())
        loader.check(L.msb_gemm_reduce_scatter(ctypes.byref(a), st), "gemm_reduce_scatter")
        lead = (x.shape[0] // ws,) + tuple(x.shape[1:-1])
        out = torch.empty(*lead, n, dtype=torch.bfloat16, device=x.device)
        own = h.ptr(h.rank, off_partial + h.rank * rows * n * 2)
        loader.check(L.msb_rs_reduce(ctypes.c_void_p(h.ptr(h.rank, off_stage)), ctypes.c_void_p(own), loader.p(out),
                                     loader.p(residual) if residual is not None else None,
                                     ctypes.c_longlong(rows), n, ws, h.rank, ctypes.c_void_p(h.ptr(h.rank, 0)),
                                     ctypes.c_uint(epoch), ctypes.c_void_p(G.status_word(x.device).data_ptr()), 0, st),
                     "rs_reduce")
        return out
