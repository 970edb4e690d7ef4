from .linear_2d import ParallelLinear2D  # noqa: F401
from .norm_2d import LayerNorm2D, RMSNorm2D  # noqa: F401
