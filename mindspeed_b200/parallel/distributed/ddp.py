"""Data-parallel wrapper with bucketed, overlapped gradient reduction (Megatron-core DDP surface).

reference: patched ``DistributedDataParallel`` hooks in mindspeed/core/data_parallel/distributed_data_parallel.py:23-142
and bucket groups in mindspeed/core/distributed/param_and_grad_buffer.py:140-239.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import parallel_state as ps
from .buffers import ParamAndGradBuffer


@dataclass
class DistributedDataParallelConfig:
    grad_reduce_in_fp32: bool = False
    quant_grads: bool = False            # gradient buffers (accumulation and reduction) in fp16 instead of fp32 / the parameter type
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    align_param_gather: bool = False
    use_distributed_optimizer: bool = False
    num_distributed_optimizer_instances: int = 1
    check_for_nan_in_grad: bool = False
    bucket_size: Optional[int] = None
    average_in_collective: bool = False
    fp8_param_gather: bool = False
    contiguous_params: bool = True
    param_and_grad_buffer_pad: Optional[int] = None
    reset_bucket_group_order: bool = False
    fused_dist_opt: bool = False      # gradient / parameter buffers in a symmetric heap; the optimizer's fused kernel moves the data


class DistributedDataParallel(nn.Module):
    def __init__(self, config, ddp_config: DistributedDataParallelConfig, module: nn.Module,
                 disable_bucketing: bool = False):
        super().__init__()
        self.config, self.ddp_config, self.module = config, ddp_config, module
        dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        if ddp_config.bucket_size is None:
            ddp_config.bucket_size = max(40_000_000, 1_000_000 * dp)
        if not ddp_config.overlap_grad_reduce:
            ddp_config.bucket_size = None
        bucket_size = None if disable_bucketing else ddp_config.bucket_size
        dense, expert = [], []
        for p in module.parameters():
            if not p.requires_grad:
                continue
            (expert if not getattr(p, "allreduce", True) else dense).append(p)
        self.buffers: List[ParamAndGradBuffer] = []
        self.expert_buffers: List[ParamAndGradBuffer] = []

        def mk(params, group, scale, out):
            by_dtype = {}
            for p in params:
                by_dtype.setdefault(p.dtype, []).append(p)
            for dt, ps_ in by_dtype.items():
                # --quant-grads: 16-bit gradient buffers halve gradient memory and reduce-scatter traffic (reference:
                # mindspeed/core/optimizer/low_precision/param_and_grad_buffer.py:23-33, dtype fp16)
                gdt = torch.float16 if ddp_config.quant_grads else (torch.float32 if ddp_config.grad_reduce_in_fp32 else dt)
                out.append(ParamAndGradBuffer(ddp_config, dt, gdt, ps_, group, bucket_size, scale))

        dp_group = ps.get_data_parallel_group(with_context_parallel=True)
        if config.calculate_per_token_loss or ddp_config.average_in_collective:
            scale, escale = 1.0, 1.0
        else:
            scale = 1.0 / dp
            escale = 1.0 / dp  # expert grads are averaged over the same number of samples
        if dense:
            mk(dense, dp_group, scale, self.buffers)
        if expert:
            edp_group = ps.get_expert_data_parallel_group()
            edp = ps.get_expert_data_parallel_world_size()
            mk(expert, edp_group, escale * 1.0, self.expert_buffers)
            for b in self.expert_buffers:
                # sum over edp ranks then scale by 1/dp overall: scaling factor applied before reduce
                b.gradient_scaling_factor = escale
        self._param_to_buffer = {}
        for buf in self.buffers + self.expert_buffers:
            for p in buf.params:
                self._param_to_buffer[id(p)] = buf
        self._hooks = []
        for p in module.parameters():
            if p.requires_grad:
                p._main_grad_ready_cb = self._on_main_grad_ready
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(p)))

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def _on_main_grad_ready(self, p):
        self._param_to_buffer[id(p)].register_grad_ready(p)

    def _make_hook(self, p):
        def hook(param):
            if param.grad is not None:
                if not getattr(param, "grad_added_to_main_grad", False):
                    param.main_grad.add_(param.grad.to(param.main_grad.dtype))
                param.grad = None
            self._param_to_buffer[id(param)].register_grad_ready(param)
        return hook

    @contextlib.contextmanager
    def no_sync(self):
        for b in self.buffers + self.expert_buffers:
            b.is_last_microbatch = False
        try:
            yield
        finally:
            for b in self.buffers + self.expert_buffers:
                b.is_last_microbatch = True

    def start_grad_sync(self, *unused):
        for buf in self.buffers + self.expert_buffers:
            for b in buf.buckets:
                buf.start_grad_sync(b)

    def finish_grad_sync(self):
        for buf in self.buffers + self.expert_buffers:
            buf.finish_grad_sync()

    def scale_gradients(self, factor: float):
        for buf in self.buffers + self.expert_buffers:
            buf.scale_gradients(factor)

    def zero_grad_buffer(self):
        for p in self.module.parameters():
            if p.requires_grad:
                p.grad_added_to_main_grad = False
        for buf in self.buffers + self.expert_buffers:
            buf.reset()

    def broadcast_params(self):
        for p in self.module.parameters():
            is_expert = not getattr(p, "allreduce", True)
            group = ps.get_expert_data_parallel_group() if is_expert else ps.get_data_parallel_group(with_context_parallel=True)
            if group is not None and dist.get_world_size(group) > 1:
                src = dist.get_global_rank(group, 0)
                dist.broadcast(p.data, src=src, group=group)

    def start_param_sync(self, *unused, force_sync=False, force_dispatch=False):
        for buf in self.buffers + self.expert_buffers:
            if buf.ddp_config.use_distributed_optimizer:
                for b in buf.buckets:
                    buf.start_param_sync(b, async_op=not force_sync and self.ddp_config.overlap_param_gather)
                if force_sync or not self.ddp_config.overlap_param_gather:
                    for b in buf.buckets:
                        buf.finish_param_sync(b)

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)

    def sharded_state_dict(self, *a, **k):
        return self.module.sharded_state_dict(*a, **k)
