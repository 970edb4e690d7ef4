"""Megatron-free parallel engine: wrap any HF-style ``nn.Module`` with tensor / expert / fully-sharded parallelism,
activation recompute, Ulysses context parallelism (engine/context_parallel.py), fp8 linears (engine/quantization.py), host-parked activations and optimizer state (engine/memory.py)
and a chunked LM loss from one config object.
reference: mindspeed/fsdp/mindspeed_parallel_engine.py:14-68 (and the near-duplicate mindspeed/lite/*)."""
from .config import MemoryPlanConfig, ParallelEngineConfig, QuantizeConfig
from .parallel_engine import MindSpeedParallelEngine
from .chunk_loss import chunked_lm_loss

__all__ = ["ParallelEngineConfig", "QuantizeConfig", "MemoryPlanConfig", "MindSpeedParallelEngine", "chunked_lm_loss"]
