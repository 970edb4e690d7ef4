from .logging import print_rank_0, print_rank_last, log_rank_0, log_warning_once, set_log_config  # noqa: F401
