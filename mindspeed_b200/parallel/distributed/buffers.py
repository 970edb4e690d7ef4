"""Contiguous parameter / gradient buffers with buckets for overlapped data-parallel communication.

All parameters of one (param dtype, is-expert) class live in one flat ``param_data`` buffer and
their fp32 (or param-dtype) gradients in one flat ``grad_data`` buffer; ``param.main_grad`` is a
view of the latter.  The buffer is cut into buckets in *reverse* parameter order (gradients become
ready back to front).  Every bucket is padded to a multiple of ``dp_size * 64`` elements so each
distributed-optimizer shard starts 128-byte aligned
(reference: mindspeed/core/distributed/param_and_grad_buffer.py:57-267 for the per-bucket async
reduce-scatter / all-reduce / next-bucket all-gather chaining; padding
mindspeed/core/distributed/buffer_pad/adaptor.py:20-263).

With 180 GB of HBM per GPU and NVSwitch collectives whose cost is not per-link bound, the default
bucket is large (``max(40M, 1M * dp)`` elements): few launches, long enough to hide behind backward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def _pad_to(n, m):
    return ((n + m - 1) // m) * m


@dataclass
class Bucket:
    index: int
    start: int  # offset in the flat buffer (elements)
    end: int    # padded end
    params: List[torch.nn.Parameter] = field(default_factory=list)
    param_ranges: Dict[int, tuple] = field(default_factory=dict)  # id(param) -> (start, end) in flat buffer
    ready: set = field(default_factory=set)
    handle: object = None
    param_handle: object = None

    @property
    def numel(self):
        return self.end - self.start


class ParamAndGradBuffer:
    def __init__(self, ddp_config, param_dtype, grad_dtype, params, dp_group, bucket_size: Optional[int],
                 gradient_scaling_factor: float = 1.0, device=None):
        self.ddp_config = ddp_config
        self.param_dtype, self.grad_dtype = param_dtype, grad_dtype
        self.dp_group = dp_group
        self.dp_size = 1 if dp_group is None else dist.get_world_size(dp_group)
        self.dp_rank = 0 if dp_group is None else dist.get_rank(dp_group)
        self.gradient_scaling_factor = gradient_scaling_factor
        self.params = list(params)
        align = self.dp_size * 64 if ddp_config.use_distributed_optimizer else 64
        if getattr(ddp_config, "pad_buckets_for_high_nccl_busbw", False) or getattr(ddp_config, "param_and_grad_buffer_pad", None):
            align = math.lcm(align, int(getattr(ddp_config, "param_and_grad_buffer_pad", None) or 2 ** 16))
        # layout: reverse order so the last layers' grads (ready first) share the first bucket
        self.buckets: List[Bucket] = []
        cur = Bucket(0, 0, 0)
        offset = 0
        self.param_index: Dict[int, tuple] = {}
        for p in reversed(self.params):
            n = p.numel()
            start = _pad_to(offset, 64)
            end = start + n
            cur.params.append(p)
            cur.param_ranges[id(p)] = (start, end)
            self.param_index[id(p)] = (start, end, len(self.buckets))
            offset = end
            if bucket_size is not None and (offset - cur.start) >= bucket_size:
                offset = _pad_to(offset, align)
                cur.end = offset
                self.buckets.append(cur)
                cur = Bucket(len(self.buckets), offset, offset)
        if cur.params:
            offset = _pad_to(offset, align)
            cur.end = offset
            self.buckets.append(cur)
        self.numel = offset
        dev = device if device is not None else self.params[0].device
        self.fused = bool(getattr(ddp_config, "fused_dist_opt", False) and ddp_config.use_distributed_optimizer
                          and 2 <= self.dp_size <= 8 and dev.type == "cuda" and param_dtype == torch.bfloat16
                          and grad_dtype in (torch.float32, torch.bfloat16))
        self.heap = None
        if self.fused:
            # both buffers live in a symmetric heap over the data-parallel group: the optimizer's fused kernel pulls
            # gradient shards from the peers and pushes updated parameters to them, so no NCCL collective touches them
            from ..symm_mem import get_heap
            gsz = torch.empty((), dtype=grad_dtype).element_size()
            ParamAndGradBuffer._heap_seq = getattr(ParamAndGradBuffer, "_heap_seq", 0) + 1
            self.heap = get_heap(dp_group, self.numel * (gsz + 2) + (1 << 20), tag=f"dp{ParamAndGradBuffer._heap_seq}")
            self.grad_off = self.heap.alloc("grad", self.numel * gsz)
            self.param_off = self.heap.alloc("param", self.numel * 2)
            self.grad_data = self.heap.tensor(self.grad_off, (self.numel,), grad_dtype)
            self.grad_data.zero_()
            self.param_data = self.heap.tensor(self.param_off, (self.numel,), param_dtype)
            self.param_data.zero_()
        else:
            self.grad_data = torch.zeros(self.numel, dtype=grad_dtype, device=dev)
            self.param_data = None
            if ddp_config.use_distributed_optimizer or ddp_config.contiguous_params:
                self.param_data = torch.zeros(self.numel, dtype=param_dtype, device=dev)
        for p in self.params:
            s, e, _ = self.param_index[id(p)]
            if self.param_data is not None:
                view = self.param_data[s:e].view(p.shape)
                view.copy_(p.data)
                p.data = view
            p.main_grad = self.grad_data[s:e].view(p.shape)
            p.grad_added_to_main_grad = False
        self.is_last_microbatch = True
        self._shard_cache = {}

    # ---- views ----
    def bucket_grad(self, b: Bucket):
        return self.grad_data[b.start:b.end]

    def bucket_param(self, b: Bucket):
        return self.param_data[b.start:b.end]

    def shard_range(self, b: Bucket):
        per = b.numel // self.dp_size
        return b.start + self.dp_rank * per, b.start + (self.dp_rank + 1) * per

    # ---- lifecycle ----
    def reset(self):
        self.grad_data.zero_()
        for b in self.buckets:
            b.ready.clear()
            b.handle = None
        self.is_last_microbatch = True

    def scale_gradients(self, factor: float):
        self.grad_data.mul_(factor)

    def register_grad_ready(self, param):
        """Called from the backward hook of ``param``; launches the bucket's collective when complete."""
        if not self.is_last_microbatch:
            return
        _, _, bi = self.param_index[id(param)]
        b = self.buckets[bi]
        b.ready.add(id(param))
        if self.ddp_config.overlap_grad_reduce and len(b.ready) == len(b.params):
            self.start_grad_sync(b)

    def start_grad_sync(self, b: Bucket):
        if self.fused:
            b.handle = "done"          # the optimizer's fused kernel reduces (and scales) straight from the peers' buffers
            return
        if b.handle is not None or self.dp_size == 1 and self.gradient_scaling_factor == 1.0:
            if self.dp_size == 1:
                b.handle = "done"
            return
        g = self.bucket_grad(b)
        if self.ddp_config.check_for_nan_in_grad:
            if not torch.isfinite(g.float().sum()):
                raise RuntimeError(f"non-finite gradient in bucket {b.index} before data-parallel reduction")
        if self.gradient_scaling_factor != 1.0:
            g.mul_(self.gradient_scaling_factor)
        if self.dp_size == 1:
            b.handle = "done"
            return
        op = dist.ReduceOp.AVG if self.ddp_config.average_in_collective else dist.ReduceOp.SUM
        async_op = self.ddp_config.overlap_grad_reduce
        if self.ddp_config.use_distributed_optimizer:
            s, e = self.shard_range(b)
            out = self.grad_data[s:e]
            if dist.get_backend(self.dp_group) == "gloo":
                if op == dist.ReduceOp.AVG:
                    g.div_(self.dp_size)
                dist.all_reduce(g, group=self.dp_group)
                b.handle = "done"
            else:
                b.handle = dist.reduce_scatter_tensor(out, g, op=op, group=self.dp_group, async_op=async_op) or "done"
        else:
            if op == dist.ReduceOp.AVG and dist.get_backend(self.dp_group) == "gloo":
                g.div_(self.dp_size)
                op = dist.ReduceOp.SUM
            b.handle = dist.all_reduce(g, op=op, group=self.dp_group, async_op=async_op) or "done"

    def finish_grad_sync(self):
        for b in self.buckets:
            if b.handle is None:
                self.start_grad_sync(b)
            if b.handle not in (None, "done"):
                b.handle.wait()
            b.handle = None
            b.ready.clear()

    # ---- parameter all-gather (distributed optimizer) ----
    def start_param_sync(self, b: Bucket, async_op=False):
        if self.dp_size == 1 or self.fused:      # fused: the optimizer kernel already pushed the new weights everywhere
            return
        s, e = self.shard_range(b)
        full = self.bucket_param(b)
        if dist.get_backend(self.dp_group) == "gloo":
            parts = list(full.chunk(self.dp_size))
            dist.all_gather(parts, self.param_data[s:e].clone(), group=self.dp_group)
            return
        b.param_handle = dist.all_gather_into_tensor(full, self.param_data[s:e], group=self.dp_group, async_op=async_op)

    def finish_param_sync(self, b: Bucket):
        if b.param_handle is not None:
            b.param_handle.wait()
            b.param_handle = None
