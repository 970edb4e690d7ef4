"""Host side of csrc/kernels/dist_opt_fused.cu: the distributed-optimizer step as peer-memory kernels.

``FusedShardedAdam(group, numel, grad_dtype)`` owns, in a symmetric heap over the data-parallel group,
    grad_buffer    the full gradient bucket of this rank (backward accumulates into it),
    param_buffer   the full bf16 parameter bucket (the model's parameters are views into it),
and locally the fp32 master / m / v of its shard.  ``step()`` runs
    no clipping    one kernel: pull-reduce gradients -> AdamW -> push new bf16 weights to every rank
    clipping       kernel 1: pull-reduce + squared norm; one scalar all-reduce; kernel 2: AdamW with the clip coefficient
                   read from device memory -> push
followed by ``wait_params()`` (bounded device-side wait) before the next forward reads the parameters.
It replaces NCCL reduce-scatter + cast/scale + Adam + NCCL all-gather of a ZeRO-1 step; results match that sequence up to
fp32 summation order (fixed rank order here, so runs are bit-reproducible).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch
import torch.distributed as dist

from . import gemm as G
from . import loader
from ..parallel.symm_mem import SymmetricHeap, get_heap


class _Args(ctypes.Structure):
    _fields_ = [("peer_grad", ctypes.c_void_p * 8), ("peer_param", ctypes.c_void_p * 8), ("reduced", ctypes.c_void_p),
                ("master", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p), ("sumsq", ctypes.c_void_p),
                ("clip_coef", ctypes.c_void_p), ("found_inf", ctypes.c_void_p), ("n", ctypes.c_longlong),
                ("shard_offset", ctypes.c_longlong), ("grad_scale", ctypes.c_float), ("lr", ctypes.c_float),
                ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float), ("wd", ctypes.c_float),
                ("step", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int), ("grad_is_bf16", ctypes.c_int),
                ("pull", ctypes.c_int), ("do_adam", ctypes.c_int), ("push", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("flag_local", ctypes.c_void_p), ("flag_peer", ctypes.c_void_p * 8), ("status", ctypes.c_void_p),
                ("wait_limit_ms", ctypes.c_int)]


class FusedShardedAdam:
    def __init__(self, group, numel: int, grad_dtype=torch.float32, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 tag: str = "dp"):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise RuntimeError("the fused optimizer step covers one NVSwitch domain (<= 8 ranks)")
        if grad_dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("gradients must be fp32 or bf16")
        div = 4 * self.world
        self.numel = ((numel + div - 1) // div) * div
        self.shard = self.numel // self.world
        self.grad_dtype = grad_dtype
        gsz = 4 if grad_dtype == torch.float32 else 2
        heap_bytes = self.numel * (gsz + 2) + (1 << 20)
        self.heap: SymmetricHeap = get_heap(group, heap_bytes, tag=tag)
        self.grad_off = self.heap.alloc("dist_opt_grad", self.numel * gsz)
        self.param_off = self.heap.alloc("dist_opt_param", self.numel * 2)
        self.grad_buffer = self.heap.tensor(self.grad_off, (self.numel,), grad_dtype)
        self.param_buffer = self.heap.tensor(self.param_off, (self.numel,), torch.bfloat16)
        self.grad_buffer.zero_()
        dev = self.grad_buffer.device
        self.master = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.reduced = torch.zeros_like(self.master)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.clip = torch.ones(1, dtype=torch.float32, device=dev)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self._last_epoch = 0

    def init_from_params(self, full_params_bf16: torch.Tensor):
        """Load the bucket (padded with zeros) and derive the fp32 master shard from it."""
        n = full_params_bf16.numel()
        self.param_buffer.zero_()
        self.param_buffer[:n].copy_(full_params_bf16.reshape(-1))
        self.master.copy_(self.param_buffer[self.rank * self.shard:(self.rank + 1) * self.shard].float())
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _launch(self, pull, do_adam, push, grad_scale, use_clip):
        L = loader.require_lib()
        h = self.heap
        a = _Args()
        for r in range(self.world):
            a.peer_grad[r] = h.ptr(r, self.grad_off)
            a.peer_param[r] = h.ptr(r, self.param_off)
            a.flag_peer[r] = h.ptr(r, 0)
        a.reduced, a.master, a.m, a.v = self.reduced.data_ptr(), self.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr()
        a.sumsq = self.sumsq.data_ptr()
        a.clip_coef = self.clip.data_ptr() if use_clip else None
        a.found_inf = None
        a.n, a.shard_offset = self.shard, self.rank * self.shard
        a.grad_scale, a.lr, a.beta1, a.beta2, a.eps, a.wd = grad_scale, self.lr, self.betas[0], self.betas[1], self.eps, self.wd
        a.step, a.world, a.rank = max(1, self.step_count), self.world, self.rank
        a.grad_is_bf16 = int(self.grad_dtype == torch.bfloat16)
        a.pull, a.do_adam, a.push = int(pull), int(do_adam), int(push)
        a.epoch = h.next_epoch()
        a.flag_local = h.ptr(h.rank, 0)
        a.status = G.status_word(self.master.device).data_ptr()
        a.wait_limit_ms = 0
        loader.check(L.msb_dist_opt_fused(ctypes.byref(a), ctypes.c_void_p(loader.stream_ptr())), "dist_opt_fused")
        self._last_epoch = a.epoch

    def step(self, grad_scale: float = 1.0, clip_grad: float = 0.0) -> Optional[torch.Tensor]:
        """``grad_scale`` multiplies the summed gradient (1 / (dp x micro-batches) for a mean).  Returns the global
        gradient norm (device scalar) when clipping is on."""
        self.step_count += 1
        self.sumsq.zero_()
        if clip_grad and clip_grad > 0:
            self._launch(pull=True, do_adam=False, push=False, grad_scale=grad_scale, use_clip=False)
            if self.world > 1:
                dist.all_reduce(self.sumsq, group=self.group)
            norm = self.sumsq.sqrt()
            torch.clamp(clip_grad / (norm + 1e-6), max=1.0, out=self.clip)
            self._launch(pull=False, do_adam=True, push=True, grad_scale=grad_scale, use_clip=True)
            self.wait_params()
            return norm
        self._launch(pull=True, do_adam=True, push=True, grad_scale=grad_scale, use_clip=False)
        self.wait_params()
        return None

    def wait_params(self):
        if self.world == 1:
            return
        L = loader.require_lib()
        h = self.heap
        loader.check(L.msb_dist_opt_wait_params(ctypes.c_void_p(h.ptr(h.rank, 0)), ctypes.c_uint(self._last_epoch), self.world,
                                                ctypes.c_void_p(G.status_word(self.master.device).data_ptr()), 0,
                                                ctypes.c_void_p(loader.stream_ptr())), "dist_opt_wait_params")

    def zero_grad(self):
        self.grad_buffer.zero_()
