"""Tensor-parallel layers: column / row parallel linear, vocab-parallel embedding.

API follows Megatron-core ``tensor_parallel.layers``.  The linear autograd functions
implement the sequence-parallel algorithm of the reference's non-fused path
(mindspeed/core/tensor_parallel/coc_feature/rewrite_parallel_linears_sequence_parallel.py:7-88):

  column fwd:  AG(x) -> total @ W^T                 bwd: AG(x) || dX_full = dY @ W -> RS(dX_full) || dW = dY^T @ total
  row    fwd:  x @ W^T -> RS                        bwd: AG(dY) -> dX = dY_full @ W ; dW = dY_full^T @ x

and delegate every "GEMM next to a collective" to the active backend of
``comm_ops`` so that the fused sm_100a kernels and the library path are
interchangeable.  The saved-tensor policy is the MC2 one
(reference: mindspeed/core/tensor_parallel/mc2_feature/linear_function.py:28-60,76-87):
only the *sharded* input is saved and re-gathered in backward.

Weight gradients can be (a) returned to autograd, (b) accumulated in place into an
fp32 ``weight.main_grad`` (``gradient_accumulation_fusion``; reference
mindspeed/ops/npu_matmul_add.py:51-66), (c) deferred through ``WeightGradStore`` so a
pipeline schedule can place them where they hide communication.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import mappings as M
from . import parallel_state as ps
from .comm_ops import get_ops
from .weight_grad_store import WeightGradStore

_MODEL_PARALLEL_ATTRIBUTE_DEFAULTS = {"tensor_model_parallel": False, "partition_dim": -1, "partition_stride": 1}


def set_tensor_model_parallel_attributes(tensor, is_parallel, dim, stride):
    setattr(tensor, "tensor_model_parallel", is_parallel)
    setattr(tensor, "partition_dim", dim)
    setattr(tensor, "partition_stride", stride)


def set_defaults_if_not_set_tensor_model_parallel_attributes(tensor):
    for k, v in _MODEL_PARALLEL_ATTRIBUTE_DEFAULTS.items():
        if not hasattr(tensor, k):
            setattr(tensor, k, v)


def copy_tensor_model_parallel_attributes(dst, src):
    for k in _MODEL_PARALLEL_ATTRIBUTE_DEFAULTS:
        if hasattr(src, k):
            setattr(dst, k, getattr(src, k))


def param_is_not_tensor_parallel_duplicate(param):
    return getattr(param, "tensor_model_parallel", False) or ps.get_tensor_model_parallel_rank() == 0


def divide(a, b):
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def _init_sharded(weight, full_rows, full_cols, partition_dim, init_method, rank, world, params_dtype, stride=1):
    """Initialise a tensor-parallel weight.

    CPU tensors: draw the *full* matrix from one RNG stream and keep this rank's slice, so any TP degree
    yields the same logical weights (what the CPU loss-curve oracle relies on).
    GPU tensors: draw only the local shard on the device under the tensor-parallel RNG stream (per-rank
    seed), as Megatron's ``_initialize_affine_weight_gpu`` does; no host-sized temporaries."""
    if weight.is_cuda:
        from .random import get_cuda_rng_tracker
        tr = get_cuda_rng_tracker()
        with torch.no_grad():
            if tr.is_initialized() and world > 1:
                with tr.fork():
                    init_method(weight)
            else:
                init_method(weight)
        return
    master = torch.empty(full_rows, full_cols, dtype=torch.float32)
    init_method(master)
    per = (full_rows if partition_dim == 0 else full_cols) // world
    per_stride = per // stride
    pieces = torch.split(master, per_stride, dim=partition_dim)
    mine = pieces[rank::world]
    with torch.no_grad():
        weight.copy_(torch.cat(mine, dim=partition_dim).to(params_dtype))


# Keep the all-gathered input of sequence-parallel column linears for backward (memory for communication): the
# reference's ``all_gather_recomputation_enabled = False`` setting (coc_feature/min_comm_cfg.py:44-54).
_KEEP_GATHERED = {"on": False}


def set_keep_gathered_input(flag: bool):
    _KEEP_GATHERED["on"] = bool(flag)


class _ColumnLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, group, sequence_parallel, allreduce_dgrad, grad_accum_fusion, wgrad_deferral):
        ops = get_ops()
        ctx.group, ctx.sp, ctx.allreduce_dgrad = group, sequence_parallel, allreduce_dgrad
        ctx.fusion, ctx.defer, ctx.use_bias = grad_accum_fusion, wgrad_deferral, bias is not None
        keep = bool(sequence_parallel and _KEEP_GATHERED["on"] and ctx.needs_input_grad[1])
        ctx.kept_total = keep
        if sequence_parallel:
            y, total = ops.allgather_matmul(x, weight, group, nt=True, need_gathered=keep)
            if keep:
                # the gathered activation is a by-product of the fused kernel: keeping it (one local copy out of the
                # recycled symmetric buffer) removes the all-gather that backward would otherwise redo for dW
                total = total.clone() if getattr(ops, "gathered_is_view", False) else total
                ctx.save_for_backward(total, weight)
            else:
                ctx.save_for_backward(x, weight)
        else:
            ctx.save_for_backward(x, weight)
        if not sequence_parallel:
            y = ops.matmul(x, weight, nt=True)
        if bias is not None:
            y = y + bias
        return y

    @staticmethod
    def backward(ctx, dy):
        ops = get_ops()
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        db = dy.reshape(-1, dy.shape[-1]).sum(0) if ctx.use_bias else None
        need_wgrad = weight.requires_grad
        total, ag_handle = x, None
        if ctx.sp and need_wgrad and not ctx.defer and not ctx.kept_total:
            total, ag_handle = M.all_gather_first_dim(x, ctx.group, async_op=True)
        concurrent = (ctx.sp and need_wgrad and not ctx.defer and ctx.kept_total and ctx.fusion and hasattr(weight, "main_grad")
                      and dy.is_cuda and getattr(ops, "concurrent_wgrad", False))
        if concurrent:
            # weight gradient on a side stream, sharing the SMs with the NVLink-bound GEMM->reduce-scatter kernel
            dx = ops.dgrad_reduce_scatter_with_wgrad(dy, weight, total, weight.main_grad, ctx.group)
            weight.grad_added_to_main_grad = True
            cb = getattr(weight, "_main_grad_ready_cb", None)
            if cb is not None:
                cb(weight)
            return dx, None, db, None, None, None, None, None
        if ctx.sp:
            dx = ops.matmul_reduce_scatter(dy, weight, ctx.group, nt=False)
        elif ctx.allreduce_dgrad:
            dx = ops.matmul_all_reduce(dy, weight, ctx.group, nt=False)
        else:
            dx = ops.matmul(dy, weight, nt=False)
        dw = None
        if need_wgrad:
            if ctx.defer and WeightGradStore.enabled():
                WeightGradStore.put(x, dy, weight, ctx.sp and not ctx.kept_total, ctx.group, ctx.fusion)
            else:
                if ag_handle is not None:
                    ag_handle.wait()
                dw = _wgrad(ops, dy, total, weight, ctx.fusion)
        return dx, dw, db, None, None, None, None, None


class _RowLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, sequence_parallel, reduce_output, grad_accum_fusion, wgrad_deferral):
        ops = get_ops()
        ctx.group, ctx.sp, ctx.fusion, ctx.defer = group, sequence_parallel, grad_accum_fusion, wgrad_deferral
        ctx.save_for_backward(x, weight)
        if sequence_parallel:
            return ops.matmul_reduce_scatter(x, weight, group, nt=True)
        if reduce_output:
            return ops.matmul_all_reduce(x, weight, group, nt=True)
        return ops.matmul(x, weight, nt=True)

    @staticmethod
    def backward(ctx, dy):
        ops = get_ops()
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        need_wgrad = weight.requires_grad
        if ctx.sp:
            dx, dy_total = ops.allgather_matmul(dy, weight, ctx.group, nt=False, need_gathered=need_wgrad)
        else:
            dx, dy_total = ops.matmul(dy, weight, nt=False), dy
        dw = None
        if need_wgrad:
            if ctx.defer and WeightGradStore.enabled():
                if getattr(ops, "gathered_is_view", False) and ctx.sp:
                    dy_total = dy_total.clone()  # the fused op's gathered buffer is recycled two calls later
                WeightGradStore.put(x, dy_total, weight, False, ctx.group, ctx.fusion)
            else:
                dw = _wgrad(ops, dy_total, x, weight, ctx.fusion)
        return dx, dw, None, None, None, None, None


def _wgrad(ops, dy, x, weight, fusion):
    """Weight gradient.  With accumulation fusion the product is added straight into the fp32
    ``weight.main_grad`` and autograd gets ``None``; the data-parallel wrapper is told through
    ``weight._main_grad_ready_cb`` (it cannot rely on the AccumulateGrad node firing)."""
    if fusion and hasattr(weight, "main_grad"):
        ops.wgrad(dy, x, weight.main_grad)
        weight.grad_added_to_main_grad = True
        cb = getattr(weight, "_main_grad_ready_cb", None)
        if cb is not None:
            cb(weight)
        return None
    return ops.wgrad(dy, x, None).to(weight.dtype)


def linear_with_grad_accumulation_and_async_allreduce(input, weight, bias, gradient_accumulation_fusion=False,
                                                      allreduce_dgrad=False, sequence_parallel=False,
                                                      grad_output_buffer=None, wgrad_deferral_limit=0, tp_group=None,
                                                      async_grad_allreduce=None):
    """Megatron-named entry to the column-linear autograd function."""
    if async_grad_allreduce is not None:
        allreduce_dgrad = async_grad_allreduce
    group = ps.get_tensor_model_parallel_group() if tp_group is None else tp_group
    return _ColumnLinearFn.apply(input, weight, bias, group, sequence_parallel, allreduce_dgrad,
                                 gradient_accumulation_fusion, False)


class ColumnParallelLinear(nn.Module):
    """Y = X A^T + b with A split along its output dimension: A = [A_1; ...; A_p]."""

    def __init__(self, input_size, output_size, *, config, init_method: Callable, bias=True, gather_output=False,
                 stride=1, keep_master_weight_for_test=False, skip_bias_add=False, skip_weight_param_allocation=False,
                 embedding_activation_buffer=None, grad_output_buffer=None, is_expert=False, tp_comm_buffer_name=None,
                 disable_grad_reduce=False, tp_group=None):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.gather_output, self.skip_bias_add, self.is_expert = gather_output, skip_bias_add, is_expert
        self.config = config
        self.disable_grad_reduce = disable_grad_reduce
        if tp_group is not None:
            self.tp_group = tp_group
        elif is_expert:
            self.tp_group = ps.get_expert_tensor_parallel_group(check_initialized=False)
        else:
            self.tp_group = ps.get_tensor_model_parallel_group(check_initialized=False)
        world = ps.get_expert_tensor_parallel_world_size() if is_expert else ps.get_tensor_model_parallel_world_size()
        rank = ps.get_expert_tensor_parallel_rank() if is_expert else ps.get_tensor_model_parallel_rank()
        self.world, self.rank = world, rank
        self.output_size_per_partition = divide(output_size, world)
        self.sequence_parallel = config.sequence_parallel and world > 1
        self.explicit_expert_comm = is_expert and (world > 1 or config.expert_model_parallel_size > 1)
        self.gradient_accumulation_fusion = config.gradient_accumulation_fusion
        self.allreduce_dgrad = world > 1 and not self.sequence_parallel and not disable_grad_reduce
        if self.explicit_expert_comm:
            self.sequence_parallel, self.allreduce_dgrad = False, False
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        if not skip_weight_param_allocation:
            self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, device=dev,
                                                   dtype=config.params_dtype))
            if config.perform_initialization:
                _init_sharded(self.weight, output_size, input_size, 0, init_method, rank, world, config.params_dtype,
                              stride)
            set_tensor_model_parallel_attributes(self.weight, True, 0, stride)
            setattr(self.weight, "allreduce", not (is_expert and self.explicit_expert_comm))
        else:
            self.weight = None
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, device=dev, dtype=config.params_dtype))
            set_tensor_model_parallel_attributes(self.bias, True, 0, stride)
            setattr(self.bias, "allreduce", not (is_expert and self.explicit_expert_comm))
        else:
            self.register_parameter("bias", None)
        self.wgrad_deferral = False

    def forward(self, input_, weight=None, runtime_gather_output=None):
        weight = self.weight if weight is None else weight
        bias = self.bias if not self.skip_bias_add else None
        y = _ColumnLinearFn.apply(input_, weight, bias, self.tp_group, self.sequence_parallel, self.allreduce_dgrad,
                                  self.gradient_accumulation_fusion, self.wgrad_deferral)
        gather = self.gather_output if runtime_gather_output is None else runtime_gather_output
        if gather and self.world > 1:
            y = M.gather_from_tensor_model_parallel_region(y, self.tp_group)
        return y, (self.bias if self.skip_bias_add else None)

    def sharded_state_dict(self, prefix="", sharded_offsets=(), metadata=None):
        from ..checkpointing.sharded import make_tp_sharded_tensors
        return make_tp_sharded_tensors(self.state_dict(prefix="", keep_vars=True), prefix, {"weight": 0, "bias": 0},
                                       sharded_offsets, self.rank, self.world)


class RowParallelLinear(nn.Module):
    """Y = X A^T + b with A split along its input dimension and X along its last dimension."""

    def __init__(self, input_size, output_size, *, config, init_method: Callable, bias=True, input_is_parallel=True,
                 skip_bias_add=False, stride=1, keep_master_weight_for_test=False, is_expert=False,
                 tp_comm_buffer_name=None, tp_group=None):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.input_is_parallel, self.skip_bias_add, self.is_expert = input_is_parallel, skip_bias_add, is_expert
        self.config = config
        if tp_group is not None:
            self.tp_group = tp_group
        elif is_expert:
            self.tp_group = ps.get_expert_tensor_parallel_group(check_initialized=False)
        else:
            self.tp_group = ps.get_tensor_model_parallel_group(check_initialized=False)
        world = ps.get_expert_tensor_parallel_world_size() if is_expert else ps.get_tensor_model_parallel_world_size()
        rank = ps.get_expert_tensor_parallel_rank() if is_expert else ps.get_tensor_model_parallel_rank()
        self.world, self.rank = world, rank
        self.input_size_per_partition = divide(input_size, world)
        self.sequence_parallel = config.sequence_parallel and world > 1
        if self.sequence_parallel and not input_is_parallel:
            raise RuntimeError("sequence parallel needs input_is_parallel=True")
        self.explicit_expert_comm = is_expert and (world > 1 or config.expert_model_parallel_size > 1)
        self.gradient_accumulation_fusion = config.gradient_accumulation_fusion
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, device=dev,
                                               dtype=config.params_dtype))
        if config.perform_initialization:
            _init_sharded(self.weight, output_size, input_size, 1, init_method, rank, world, config.params_dtype, stride)
        set_tensor_model_parallel_attributes(self.weight, True, 1, stride)
        setattr(self.weight, "allreduce", not (is_expert and self.explicit_expert_comm))
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, device=dev, dtype=config.params_dtype))
            setattr(self.bias, "allreduce", not (is_expert and self.explicit_expert_comm))
            setattr(self.bias, "sequence_parallel", self.sequence_parallel)
        else:
            self.register_parameter("bias", None)
        self.wgrad_deferral = False

    def forward(self, input_):
        if not self.input_is_parallel:
            input_ = M.scatter_to_tensor_model_parallel_region(input_, self.tp_group)
        sp = self.sequence_parallel and not self.explicit_expert_comm
        reduce_out = self.world > 1 and not sp and not self.explicit_expert_comm
        y = _RowLinearFn.apply(input_, self.weight, self.tp_group, sp, reduce_out, self.gradient_accumulation_fusion,
                               self.wgrad_deferral)
        if self.skip_bias_add:
            return y, self.bias
        if self.bias is not None:
            y = y + self.bias
        return y, None

    def sharded_state_dict(self, prefix="", sharded_offsets=(), metadata=None):
        from ..checkpointing.sharded import make_tp_sharded_tensors
        return make_tp_sharded_tensors(self.state_dict(prefix="", keep_vars=True), prefix, {"weight": 1},
                                       sharded_offsets, self.rank, self.world)


class VocabUtility:
    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition, rank, world_size):
        return rank * per_partition, (rank + 1) * per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab, rank, world_size):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab, world_size), rank, world_size)


class VocabParallelEmbedding(nn.Module):
    """Embedding split along the vocabulary.  Out-of-range ids are masked to row 0 and their
    output rows zeroed before the reduction (reference: mindspeed/core/tensor_parallel/vocab_parallel/vocab_parallel.py:22-56)."""

    def __init__(self, num_embeddings, embedding_dim, *, init_method, reduce_scatter_embeddings=False, config, tp_group=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.reduce_scatter_embeddings = reduce_scatter_embeddings
        self.tp_group = tp_group if tp_group is not None else ps.get_tensor_model_parallel_group(check_initialized=False)
        self.world = ps.get_tensor_model_parallel_world_size()
        self.rank = ps.get_tensor_model_parallel_rank()
        self.vocab_start_index, self.vocab_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, self.rank, self.world)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.deterministic_mode = config.deterministic_mode
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim, device=dev,
                                               dtype=config.params_dtype))
        if config.perform_initialization:
            _init_sharded(self.weight, num_embeddings, embedding_dim, 0, init_method, self.rank, self.world,
                          config.params_dtype)
        set_tensor_model_parallel_attributes(self.weight, True, 0, 1)

    def forward(self, input_):
        if self.world > 1:
            mask = (input_ < self.vocab_start_index) | (input_ >= self.vocab_end_index)
            masked = (input_ - self.vocab_start_index).masked_fill(mask, 0)
        else:
            masked = input_
        out = F.embedding(masked, self.weight)
        if self.world > 1:
            out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        if self.reduce_scatter_embeddings:
            out = out.transpose(0, 1).contiguous()  # [b,s,h] -> [s,b,h]
            return M.reduce_scatter_to_sequence_parallel_region(out, self.tp_group)
        return M.reduce_from_tensor_model_parallel_region(out, self.tp_group)

    def sharded_state_dict(self, prefix="", sharded_offsets=(), metadata=None):
        from ..checkpointing.sharded import make_tp_sharded_tensors
        return make_tp_sharded_tensors(self.state_dict(prefix="", keep_vars=True), prefix, {"weight": 0},
                                       sharded_offsets, self.rank, self.world)


def linear_classes(config):
    """(column, row) linear classes for model code: the fp8-capable subclasses when an fp8 format is configured
    (they behave exactly like the plain ones outside an fp8 autocast region)."""
    if getattr(config, "fp8", None) or getattr(config, "fp8_format", None):
        from ..models.te_compat import TEColumnParallelLinear, TERowParallelLinear
        return TEColumnParallelLinear, TERowParallelLinear
    return ColumnParallelLinear, RowParallelLinear
