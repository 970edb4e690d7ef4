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
    ignored_modules: List[str] = dataclasses.field(default_factory=list)      # kept whole on every rank, gradients all-reduced
    shard_size: Optional[int] = None
    zero1_over_replicas: bool = False
    param_dtype: Optional[str] = None
    reduce_dtype: Optional[str] = "float32"


@dataclasses.dataclass
class QuantizeConfig:
    """Which linears compute in fp8 and how (reference: QuantizeConfig, mindspeed/fsdp/parallel_engine_config.py:43-66;
    recipes mindspeed/fsdp/quantization/config.py).  ``recipe_name``: "mxfp8" (32-element blocks with power-of-two scales,
    every operand quantised along the axis its GEMM contracts over), "fp8-block" (1x128 / 128x128 blocks, the tcgen05
    block-scaled kernel on a GPU), "fp8-tensorwise", "fp8-delayed".  ``apply_modules`` / ``ignored_modules``: patterns over
    qualified module names (``*`` within a dotted segment, ``**`` across); empty ``apply_modules`` = every ``nn.Linear``."""
    recipe_name: str = "mxfp8"
    apply_modules: List[str] = dataclasses.field(default_factory=list)
    ignored_modules: List[str] = dataclasses.field(default_factory=lambda: ["**lm_head**", "**embed**"])
    fp8_format: str = "hybrid"

    RECIPES = {"mxfp8": "mxfp8", "fp8-block": "blockwise", "fp8-tensorwise": "tensorwise", "fp8-delayed": "delayed"}

    def recipe(self):
        from ..models.te_compat import RECIPES
        if self.recipe_name not in self.RECIPES:
            raise ValueError(f"unknown quantisation recipe {self.recipe_name!r}; choose from {sorted(self.RECIPES)}")
        return RECIPES[self.RECIPES[self.recipe_name]](fp8_format=self.fp8_format)


@dataclasses.dataclass
class MemoryPlanConfig:
    """``swap_activation_modules``: patterns of modules whose saved-for-backward tensors wait in pinned host memory
    (reference: mindspeed/fsdp/memory/swap_activation/tensor_swap_manager.py); ``swap_optimizer``: optimizer state lives in
    pinned host memory between steps and visits the device one parameter group slice at a time
    (reference: mindspeed/fsdp/memory/swap_optimizer/swap_optimizer.py)."""
    swap_activation_modules: List[str] = dataclasses.field(default_factory=list)
    swap_min_bytes: int = 1 << 20
    swap_optimizer: bool = False
    swap_optimizer_chunk_bytes: int = 256 << 20


@dataclasses.dataclass
class ParallelEngineConfig:
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    fully_shard_parallel_size: Optional[int] = None      # None: world / tp
    ulysses_parallel_size: int = 1                       # sequence slices per data-parallel group (engine/context_parallel.py)
    tp_plan: TPPlanConfig = dataclasses.field(default_factory=TPPlanConfig)
    ep_plan: EPPlanConfig = dataclasses.field(default_factory=EPPlanConfig)
    fsdp_plan: FSDPPlanConfig = dataclasses.field(default_factory=FSDPPlanConfig)
    recompute_modules: List[str] = dataclasses.field(default_factory=list)
    loss_chunk_size: Optional[int] = None                # tokens per chunk of the LM loss; None = unchunked
    quantization: Optional[object] = None                # None | a recipe name (see QuantizeConfig) | QuantizeConfig
    memory_plan: MemoryPlanConfig = dataclasses.field(default_factory=MemoryPlanConfig)

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
        cp = self.ulysses_parallel_size
        if cp < 1 or dp % cp != 0:
            raise ValueError(f"ulysses_parallel_size {cp} must divide world / tp = {dp}")
        for pat, kind in self.tp_plan.rules.items():
            if kind not in ("colwise", "rowwise", "vocab"):
                raise ValueError(f"tp plan rule {pat!r}: unknown style {kind!r}")
        if isinstance(self.quantization, str):
            self.quantization = QuantizeConfig(recipe_name=self.quantization)
        if self.quantization is not None:
            if not isinstance(self.quantization, QuantizeConfig):
                raise ValueError("quantization is a recipe name or a QuantizeConfig")
            self.quantization.recipe()
        return self
