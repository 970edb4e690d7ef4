from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class OptimizerConfig:
    """Megatron-core ``OptimizerConfig`` fields plus the reference's additions
    (optimizer selection, EMA, swap / low-precision state flags)."""
    optimizer: str = "adam"
    lr: Optional[float] = None
    min_lr: Optional[float] = None
    decoupled_lr: Optional[float] = None
    decoupled_min_lr: Optional[float] = None
    weight_decay: float = 0.01
    fp16: bool = False
    bf16: bool = False
    params_dtype: torch.dtype = torch.float32
    use_precision_aware_optimizer: bool = False
    loss_scale: Optional[float] = None
    initial_loss_scale: float = 2 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: float = 1000
    hysteresis: int = 2
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    sgd_momentum: float = 0.9
    use_distributed_optimizer: bool = False
    overlap_param_gather_with_optimizer_step: bool = False
    clip_grad: float = 1.0
    log_num_zeros_in_grad: bool = False
    barrier_with_L1_time: bool = False
    timers: object = None
    config_logger_dir: str = ""
    # reference additions
    optimizer_selection: str = "fused_adamw"
    use_ema: bool = False
    ema_decay: float = 0.9999
    swap_optimizer: bool = False
    swap_optimizer_times: int = 16
    quant_states: Optional[str] = None
    reuse_fp32_param: bool = False
    compress_optimizer: bool = False
