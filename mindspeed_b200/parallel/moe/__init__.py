from .moe_layer import MoELayer  # noqa: F401
from .router import TopKRouter  # noqa: F401
