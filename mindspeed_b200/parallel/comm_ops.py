"""Backend switch for "GEMM next to a collective".

The tensor-parallel linear layers are written once against this small contract
(the reference has the same seam in its TE-compatible layer:
mindspeed/te/pytorch/module/ops/comm_overlap_ops.py:37-55 with ``DefaultOps`` in
ops/default_ops.py:7-60 and the fused vendor ``Mc2Ops`` in ops/mc2_ops.py:12-79):

  allgather_matmul(x_shard, w, group, nt)      -> (y, x_total | None)
  matmul_reduce_scatter(x, w, group, nt)       -> y_shard
  matmul_all_reduce(x, w, group, nt)           -> y
  matmul(x, w, nt)                             -> y
  wgrad(dy, x, main_grad)                      -> dW (or None when accumulated in place)

``nt=True``  : y = x @ w.T   (forward of a linear whose weight is [out, in])
``nt=False`` : y = x @ w     (data-gradient of the same linear)

``DefaultOps`` is the library path (cuBLAS through torch.matmul + NCCL/gloo
collective); it is optimisation level 0 and also the CPU path.  ``ChunkedOps``
pipelines the same library calls in row chunks (the reference's CoC software
pipelining, mindspeed/core/tensor_parallel/coc_feature/coc_utils.py:113-248).
``FusedOps`` runs the sm_100a kernels that move tiles over NVLink from inside
the GEMM (mindspeed_b200/ops/fused_comm.py).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import mappings as M


def _flat2d(x):
    return x.reshape(-1, x.shape[-1])


class DefaultOps:
    name = "default"

    @staticmethod
    def matmul(x, w, nt=True):
        return torch.matmul(x, w.t() if nt else w)

    @staticmethod
    def allgather_matmul(x, w, group, nt=True, need_gathered=False):
        total = M.all_gather_first_dim(x, group)
        y = torch.matmul(total, w.t() if nt else w)
        return y, (total if need_gathered else None)

    @staticmethod
    def matmul_reduce_scatter(x, w, group, nt=True):
        y = torch.matmul(x, w.t() if nt else w)
        return M.reduce_scatter_first_dim(y, group)

    @staticmethod
    def matmul_all_reduce(x, w, group, nt=True):
        y = torch.matmul(x, w.t() if nt else w).contiguous()
        M.all_reduce(y, group)
        return y

    @staticmethod
    def wgrad(dy, x, main_grad: Optional[torch.Tensor] = None):
        """dW[out,in] = dy[tokens,out]^T @ x[tokens,in]; accumulated into main_grad when given."""
        dy2, x2 = _flat2d(dy), _flat2d(x)
        if main_grad is None:
            return torch.matmul(dy2.t(), x2)
        if main_grad.dtype == dy2.dtype:
            main_grad.addmm_(dy2.t(), x2)
        else:
            main_grad.add_(torch.matmul(dy2.t(), x2).to(main_grad.dtype))
        return None


class ChunkedOps(DefaultOps):
    """Library GEMM and collective pipelined over ``parallel_num`` row chunks.

    communicate-first for all-gather (chunk i's gather flies while chunk i-1
    multiplies), compute-first for reduce-scatter / all-reduce (chunk i's
    collective flies while chunk i+1 multiplies).
    """
    name = "chunked"
    parallel_num = 2

    @classmethod
    def _num(cls, rows):
        n = cls.parallel_num
        return 1 if rows < n or rows % n != 0 else n

    @classmethod
    def allgather_matmul(cls, x, w, group, nt=True, need_gathered=False):
        ws = dist.get_world_size(group) if group is not None else 1
        n = cls._num(x.shape[0])
        if ws == 1 or n == 1:
            return DefaultOps.allgather_matmul(x, w, group, nt, need_gathered)
        chunks = x.chunk(n, dim=0)
        per = chunks[0].shape[0]
        wt = w.t() if nt else w
        outs, handles, gathered = [None] * n, [], []
        for c in chunks:
            g, h = M.all_gather_first_dim(c, group, async_op=True)
            gathered.append(g)
            handles.append(h)
        for i in range(n):
            handles[i].wait()
            outs[i] = torch.matmul(gathered[i], wt)
        # chunk i holds rows [rank r][chunk i] for every r: interleave back to rank-major order
        def reorder(parts):
            st = torch.stack([p.reshape(ws, per, *p.shape[1:]) for p in parts], dim=1)  # [ws, n, per, ...]
            return st.reshape(ws * n * per, *parts[0].shape[1:])
        y = reorder(outs)
        return y, (reorder(gathered) if need_gathered else None)

    @classmethod
    def matmul_reduce_scatter(cls, x, w, group, nt=True):
        ws = dist.get_world_size(group) if group is not None else 1
        rows = x.shape[0]
        n = cls._num(rows // max(ws, 1))
        if ws == 1 or n == 1:
            return DefaultOps.matmul_reduce_scatter(x, w, group, nt)
        wt = w.t() if nt else w
        per = rows // ws // n
        xv = x.reshape(ws, n, per, *x.shape[1:])
        outs, handles = [], []
        for i in range(n):
            xi = xv[:, i].reshape(ws * per, *x.shape[1:])
            yi = torch.matmul(xi, wt)
            o, h = M.reduce_scatter_first_dim(yi, group, async_op=True)
            outs.append(o)
            handles.append(h)
        for h in handles:
            if h is not None:
                h.wait()
        return torch.cat(outs, dim=0)

    @classmethod
    def matmul_all_reduce(cls, x, w, group, nt=True):
        ws = dist.get_world_size(group) if group is not None else 1
        n = cls._num(x.shape[0])
        if ws == 1 or n == 1:
            return DefaultOps.matmul_all_reduce(x, w, group, nt)
        wt = w.t() if nt else w
        outs, handles = [], []
        for c in x.chunk(n, dim=0):
            y = torch.matmul(c, wt).contiguous()
            handles.append(M.all_reduce(y, group, async_op=True))
            outs.append(y)
        for h in handles:
            h.wait()
        return torch.cat(outs, dim=0)


class Sm100Ops(DefaultOps):
    """Library collectives, hand-written tcgen05 GEMMs (optimisation level >= 1 on a GPU)."""
    name = "sm100"

    @staticmethod
    def _ok(x, w):
        from ..ops import gemm as G
        return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and G.supported(x, w)
                and w.is_contiguous() and G.shapes_ok(x.numel() // x.shape[-1], w.shape[0], w.shape[1]))

    @classmethod
    def matmul(cls, x, w, nt=True):
        from ..ops import gemm as G
        if cls._ok(x, w):
            return G.linear_fwd(x, w) if nt else G.linear_dgrad(x, w)
        return DefaultOps.matmul(x, w, nt)

    @classmethod
    def allgather_matmul(cls, x, w, group, nt=True, need_gathered=False):
        total = M.all_gather_first_dim(x, group)
        return cls.matmul(total, w, nt), (total if need_gathered else None)

    @classmethod
    def matmul_reduce_scatter(cls, x, w, group, nt=True):
        return M.reduce_scatter_first_dim(cls.matmul(x, w, nt), group)

    @classmethod
    def matmul_all_reduce(cls, x, w, group, nt=True):
        y = cls.matmul(x, w, nt).contiguous()
        M.all_reduce(y, group)
        return y

    @classmethod
    def wgrad(cls, dy, x, main_grad=None):
        from ..ops import gemm as G
        dy2, x2 = _flat2d(dy), _flat2d(x)
        ok = (dy2.is_cuda and dy2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and G.supported(dy2, x2, main_grad)
              and G.shapes_ok(dy2.shape[0], dy2.shape[1], x2.shape[1])
              and (main_grad is None or (main_grad.dtype == torch.float32 and main_grad.is_contiguous())))
        if ok:
            return G.linear_wgrad(dy2, x2, main_grad)
        return DefaultOps.wgrad(dy, x, main_grad)


_ACTIVE = {"ops": DefaultOps}


def set_ops(ops) -> None:
    _ACTIVE["ops"] = ops


def get_ops():
    return _ACTIVE["ops"]


def select_ops(optimization_level: int = 0, use_fused: bool = False, use_chunked: bool = False, parallel_num: int = 2):
    """Choose the backend from flags: fused kernels (``--use-ascend-mc2`` / ``--coc-fused-kernel``
    equivalents) at level 2 on a GPU, chunk pipelining for ``--use-ascend-coc``, else the library path."""
    if use_fused and optimization_level >= 2 and torch.cuda.is_available():
        from ..ops.fused_comm import FusedOps
        set_ops(FusedOps)
    elif use_chunked:
        ChunkedOps.parallel_num = parallel_num
        set_ops(ChunkedOps)
    elif optimization_level >= 1 and torch.cuda.is_available():
        set_ops(Sm100Ops)
    else:
        set_ops(DefaultOps)
    return get_ops()
