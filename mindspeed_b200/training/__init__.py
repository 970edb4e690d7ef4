from .arguments import parse_args, validate_args, core_transformer_config_from_args  # noqa: F401
from .global_vars import get_args, get_timers, get_num_microbatches  # noqa: F401
from .initialize import initialize_megatron  # noqa: F401
from .training import pretrain, train, train_step, setup_model_and_optimizer, get_model  # noqa: F401
