"""``MindSpeedParallelEngine(config, model)``: apply, in order, quantisation -> tensor parallel plan -> expert
parallel sharding -> activation recompute -> fully sharded data parallel to an arbitrary ``nn.Module``.

Rank layout (world = dp x tp, tp innermost so a tensor-parallel group sits on adjacent GPUs of one NVSwitch
domain): rank = dp_index * tp + tp_index.  Expert-parallel groups are contiguous runs of ``ep`` data-parallel
indices at a fixed tp index; fully-sharded groups are formed the same way from ``fully_shard_parallel_size``.
reference: mindspeed/fsdp/mindspeed_parallel_engine.py:14-68.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel.distributed.fsdp import FSDPPlan, FullyShardedDataParallel
from ..parallel.random import checkpoint as _checkpoint
from .chunk_loss import chunked_lm_loss
from .config import ParallelEngineConfig
from .expert_parallel import shard_experts
from .tp_plan import apply_tp_plan
from ..utils.patterns import match as _match


class _Recompute(nn.Module):
    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner

    def forward(self, *args, **kw):
        if not torch.is_grad_enabled() or kw:
            return self.inner(*args, **kw)
        return _checkpoint(self.inner, False, *args)


class MindSpeedParallelEngine(nn.Module):
    def __init__(self, config: ParallelEngineConfig, model: nn.Module):
        super().__init__()
        self.config = config
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        config.validate(world)
        tp, ep = config.tensor_parallel_size, config.expert_parallel_size
        dp = world // tp
        self.tp_group = self.ep_group = None
        self.dp_ranks: List[int] = [rank]
        if world > 1:
            for d in range(dp):
                ranks = list(range(d * tp, (d + 1) * tp))
                g = dist.new_group(ranks) if tp > 1 else None
                if rank in ranks:
                    self.tp_group = g
            for t in range(tp):
                ranks = list(range(t, world, tp))
                if rank in ranks:
                    self.dp_ranks = ranks
                for i in range(0, dp, ep):
                    sub = ranks[i:i + ep]
                    g = dist.new_group(sub) if ep > 1 else None
                    if rank in sub:
                        self.ep_group = g
        # Ulysses context parallelism: runs of ``ulysses_parallel_size`` consecutive data-parallel indices hold slices of one
        # sequence; they stay data-parallel for gradients (every rank sees different tokens)
        self.cp_group = None
        cp = config.ulysses_parallel_size
        if world > 1 and cp > 1:
            for t in range(tp):
                ranks = list(range(t, world, tp))
                for i in range(0, dp, cp):
                    sub = ranks[i:i + cp]
                    g = dist.new_group(sub)
                    if rank in sub:
                        self.cp_group = g
        self.stats = {}
        if config.quantization is not None:
            from .quantization import convert_linears
            self.stats["quantized"] = convert_linears(model, config.quantization)
        if config.memory_plan.swap_activation_modules:
            from .memory import swap_activations
            self.stats["swap_activation"] = swap_activations(model, config.memory_plan.swap_activation_modules,
                                                             config.memory_plan.swap_min_bytes)
        self.stats["tp_modules"] = apply_tp_plan(model, config.tp_plan.rules, self.tp_group, config.tp_plan.sequence_parallel) \
            if tp > 1 else 0
        self.stats["ep_blocks"] = shard_experts(model, config.ep_plan.moe_modules, self.ep_group) \
            if ep > 1 and config.ep_plan.moe_modules else 0
        self.stats["recompute"] = self._wrap_recompute(model, config.recompute_modules)
        fs = config.fully_shard_parallel_size or dp
        self.expert_fsdp = None
        if world > 1 and (config.fsdp_plan.wrap or fs > 1):
            if self.stats["ep_blocks"]:
                # expert parameters differ between expert-parallel ranks: they are sharded / averaged over the ranks that
                # hold the same experts (stride ep inside the data-parallel group) and wrapped before the dense part
                eplan = FSDPPlan(wrap=("**.experts.*", "experts.*"), reduce_dtype=config.fsdp_plan.reduce_dtype,
                                 param_dtype=config.fsdp_plan.param_dtype)
                self.expert_fsdp = FullyShardedDataParallel(model, eplan, shard_group=self._edp_group(world, tp, dp, ep, rank) or "local",
                                                            replica_group=None, grad_scale=1.0 / ep, root_unit=False)
            plan = FSDPPlan(wrap=tuple(config.fsdp_plan.wrap), ignore=tuple(config.fsdp_plan.ignored_modules), shard_size=fs, zero1_over_replicas=config.fsdp_plan.zero1_over_replicas,
                            param_dtype=config.fsdp_plan.param_dtype, reduce_dtype=config.fsdp_plan.reduce_dtype)
            self.model = FullyShardedDataParallel(model, plan, dp_group_ranks=self.dp_ranks,
                                                  all_dp_rank_lists=[list(range(t, world, tp)) for t in range(tp)])
            self.sharded = True
        else:
            self.model = model
            self.sharded = False

    @staticmethod
    def _edp_group(world, tp, dp, ep, rank):
        """Group of the ranks that hold the same experts as ``rank`` (same tp index, dp index congruent mod ep)."""
        mine = None
        for t in range(tp):
            ranks = list(range(t, world, tp))
            for j in range(ep):
                sub = ranks[j::ep]
                g = dist.new_group(sub) if len(sub) > 1 else None
                if rank in sub:
                    mine = g
        return mine

    @staticmethod
    def _wrap_recompute(model: nn.Module, patterns: List[str]) -> int:
        n = 0
        for name, mod in list(model.named_modules()):
            if name and any(_match(name, p) or type(mod).__name__ == p for p in patterns):
                parent = model
                parts = name.split(".")
                for p in parts[:-1]:
                    parent = getattr(parent, p)
                if isinstance(getattr(parent, parts[-1]), _Recompute):
                    continue
                setattr(parent, parts[-1], _Recompute(mod))
                n += 1
        return n

    def forward(self, *a, **kw):
        if self.cp_group is not None:
            from .context_parallel import ulysses_attention_patch
            with ulysses_attention_patch(self.cp_group):
                return self.model(*a, **kw)
        return self.model(*a, **kw)

    def shard_sequence(self, x, dim: int = 1):
        """This rank's slice of a full-sequence input (tokens, labels, position ids) under Ulysses context parallelism."""
        if self.cp_group is None:
            return x
        from .context_parallel import shard_sequence
        return shard_sequence(x, self.cp_group, dim)

    def loss(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
        """LM loss from final hidden states; chunked when ``loss_chunk_size`` is set."""
        return chunked_lm_loss(hidden, lm_head_weight, labels, self.config.loss_chunk_size, ignore_index)

    def optimizer_params(self):
        if self.sharded:
            extra = self.expert_fsdp.optimizer_params() if self.expert_fsdp is not None else []
            return self.model.optimizer_params() + extra
        return [p for p in self.model.parameters() if p.requires_grad]

    def finish_grad_sync(self):
        if self.sharded:
            if self.expert_fsdp is not None:
                self.expert_fsdp.finish_grad_sync()
            self.model.finish_grad_sync()

    def wrap_optimizer(self, optimizer):
        """Apply the memory plan to an optimizer built over ``optimizer_params()``: with ``swap_optimizer`` its state is kept
        in pinned host memory between steps."""
        if self.config.memory_plan.swap_optimizer:
            from .memory import HostStateOptimizer
            return HostStateOptimizer(optimizer, self.config.memory_plan.swap_optimizer_chunk_bytes)
        return optimizer

    def post_step(self):
        if self.sharded:
            self.model.post_step()

    def zero_grad(self, set_to_none=True):
        if self.sharded:
            self.model.zero_grad(set_to_none)
            if self.expert_fsdp is not None:
                self.expert_fsdp.zero_grad(set_to_none)
        else:
            for p in self.model.parameters():
                p.grad = None
