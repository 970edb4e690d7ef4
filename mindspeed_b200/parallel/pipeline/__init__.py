from .schedules import get_forward_backward_func, forward_backward_no_pipelining  # noqa: F401
