"""mindspeed_b200: a Blackwell-native large-model training framework.

Megatron-core-compatible surface (parallel_state, TransformerConfig, GPTModel, pretrain) on PyTorch,
with the hot paths as hand-written sm_100a kernels (mindspeed_b200/csrc) and NCCL over NVLink for
plumbing.  ``--optimization-level 0`` runs library GEMM + NCCL everywhere and is the comparison baseline.
"""
__version__ = "0.1.0"
