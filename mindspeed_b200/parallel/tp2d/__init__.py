from .linear_2d import ParallelLinear2D  # noqa: F401
from .norm_2d import LayerNorm2D, RMSNorm2D  # noqa: F401
from .layers_2d import MLP2D, SelfAttention2D, from_2d_layout, to_2d_layout  # noqa: F401
