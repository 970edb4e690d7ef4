from .config import OptimizerConfig  # noqa: F401
from .adamw import AdamW, FusedTorchAdamW  # noqa: F401
from .distrib_optimizer import DistributedOptimizer, get_megatron_optimizer  # noqa: F401
