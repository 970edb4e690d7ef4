"""Megatron-free parallel engine: wrap any HF-style ``nn.Module`` with tensor / expert / fully-sharded parallelism,
activation recompute and a chunked LM loss from one config object.
reference: mindspeed/fsdp/mindspeed_parallel_engine.py:14-68 (and the near-duplicate mindspeed/lite/*)."""
from .config import ParallelEngineConfig
from .parallel_engine import MindSpeedParallelEngine
from .chunk_loss import chunked_lm_loss

__all__ = ["ParallelEngineConfig", "MindSpeedParallelEngine", "chunked_lm_loss"]
