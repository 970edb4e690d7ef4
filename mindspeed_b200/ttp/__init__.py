from .adaptor import classify_exception, install_ttp, maybe_inject_fault, ttp_exception_handler  # noqa: F401
from .controller import TTPController  # noqa: F401
from .processor import TTPPause, TTPProcessor  # noqa: F401
from .replica import build_replica_groups, select_dump_ranks  # noqa: F401
