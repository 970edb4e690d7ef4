"""Configuration of the Megatron-free engine (reference: mindspeed/fsdp/parallel_engine_config.py:9-155)."""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional


@dataclasses.dataclass
class TPPlanConfig:
    """Pattern (fnmatch over qualified module names) -> "colwise" | "rowwise" | "vocab" (embedding rows)."""
    rules: Dict[str, str] = dataclasses.field(default_factory=dict)
    sequence_parallel: bool = False


@dataclasses.dataclass
class EPPlanConfig:
    """``moe_modules``: patterns of MoE blocks exposing ``experts`` (ModuleList), ``gate`` / ``router`` (Linear to
    num_experts logits) and ``top_k``."""
    moe_modules: List[str] = dataclasses.field(default_factory=list)
    dispatcher: str = "alltoall"


@dataclasses.dataclass
class FSDPPlanConfig:
    wrap: List[str] = dataclasses.field(default_factory=list)
    shard_size: Optional[int] = None
    zero1_over_replicas: bool = False
    param_dtype: Optional[str] = None
    reduce_dtype: Optional[str] = "float32"


@dataclasses.dataclass
class ParallelEngineConfig:
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    fully_shard_parallel_size: Optional[int] = None      # None: world / tp
    tp_plan: TPPlanConfig = dataclasses.field(default_factory=TPPlanConfig)
    ep_plan: EPPlanConfig = dataclasses.field(default_factory=EPPlanConfig)
    fsdp_plan: FSDPPlanConfig = dataclasses.field(default_factory=FSDPPlanConfig)
    recompute_modules: List[str] = dataclasses.field(default_factory=list)
    loss_chunk_size: Optional[int] = None                # tokens per chunk of the LM loss; None = unchunked
    quantization: Optional[str] = None                   # None | "fp8-block" (block-scaled fp8 fake-quant linears)

    def validate(self, world_size: int):
        tp, ep = self.tensor_parallel_size, self.expert_parallel_size
        if world_size % tp != 0:
            raise ValueError(f"tensor_parallel_size {tp} must divide the world size {world_size}")
        dp = world_size // tp
        if dp % ep != 0:
            raise ValueError(f"expert_parallel_size {ep} must divide world / tp = {dp}")
        fs = self.fully_shard_parallel_size or dp
        if dp % fs != 0:
            raise ValueError(f"fully_shard_parallel_size {fs} must divide world / tp = {dp}")
        for pat, kind in self.tp_plan.rules.items():
            if kind not in ("colwise", "rowwise", "vocab"):
                raise ValueError(f"tp plan rule {pat!r}: unknown style {kind!r}")
        if self.quantization not in (None, "fp8-block"):
            raise ValueError(f"unknown quantization {self.quantization!r}")
        return self
