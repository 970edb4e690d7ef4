"""Process-wide singletons: args, timers, microbatch calculator."""
import time

_ARGS = None
_TIMERS = None
_NUM_MICROBATCHES = None


def set_args(args):
    global _ARGS
    _ARGS = args


def get_args():
    if _ARGS is None:
        raise RuntimeError("arguments are not initialised")
    return _ARGS


def get_num_microbatches():
    a = get_args()
    sizes = get_micro_batch_sizes()
    if sizes:
        return len(sizes)
    return a.global_batch_size // (a.micro_batch_size * a.data_parallel_size)


def get_micro_batch_sizes():
    """``--optimized-mbs-list``: the batch size of every micro-batch of a step (their sum times the data-parallel size is the
    global batch), or None when all micro-batches have ``--micro-batch-size`` samples."""
    a = get_args()
    sizes = getattr(a, "optimized_mbs_list", None)
    return list(sizes) if sizes and getattr(a, "optimized_mbs_mode", True) else None


class _Timer:
    def __init__(self, name):
        self.name, self.elapsed_, self.started, self.t0 = name, 0.0, False, 0.0

    def start(self, barrier=False):
        self.t0, self.started = time.time(), True

    def stop(self, barrier=False):
        if self.started:
            self.elapsed_ += time.time() - self.t0
            self.started = False

    def elapsed(self, reset=True):
        e = self.elapsed_
        if reset:
            self.elapsed_ = 0.0
        return e


class Timers:
    def __init__(self):
        self.timers = {}

    def __call__(self, name, log_level=None):
        if name not in self.timers:
            self.timers[name] = _Timer(name)
        return self.timers[name]

    def log(self, names, normalizer=1.0):
        from ..utils.logging import print_rank_last
        s = "time (ms)"
        for n in names:
            if n in self.timers:
                s += f" | {n}: {self.timers[n].elapsed() * 1000.0 / normalizer:.2f}"
        print_rank_last(s)


def get_timers():
    global _TIMERS
    if _TIMERS is None:
        _TIMERS = Timers()
    return _TIMERS
