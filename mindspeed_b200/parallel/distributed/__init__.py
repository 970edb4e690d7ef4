from .ddp import DistributedDataParallel, DistributedDataParallelConfig  # noqa: F401
from .finalize import finalize_model_grads  # noqa: F401
