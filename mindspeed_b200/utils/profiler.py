"""Step-window profiler for the training loop.

``build_profiler(args)`` returns a context manager with a ``step()`` method.  Between
``--profile-step-start`` and ``--profile-step-end`` it records with ``torch.profiler`` (Kineto / CUPTI when a GPU
is present, CPU activity otherwise) and writes one Chrome trace per rank into ``--profile-save-path``; outside the
window it costs one integer compare per step.  Levels select how much is recorded:

  level0  GPU kernels only          level1  + CPU operators         level2  + shapes, stacks, memory

In addition to the trace, a per-kernel table (name, calls, total device time, share) is written as text so that
a run on a box without a trace viewer still leaves something readable, and the count of this library's own
kernel launches during the window is appended to it.
reference: mindspeed/functional/profile/adaptor.py:13-78 (torch_npu.profiler wrapped around train()).
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class StepWindowProfiler:
    def __init__(self, start: int, end: int, save_path: str, rank: int = 0, level: str = "level0", with_cpu: bool = False,
                 with_stack: bool = False, with_memory: bool = False, record_shapes: bool = False):
        if end <= start:
            raise ValueError("profile window must satisfy end > start")
        self.start, self.end, self.save_path, self.rank = start, end, save_path, rank
        self.level = level
        self.with_cpu = with_cpu or level in ("level1", "level2")
        self.with_stack = with_stack or level == "level2"
        self.with_memory = with_memory or level == "level2"
        self.record_shapes = record_shapes or level == "level2"
        self._step = 0
        self._prof: Optional[torch.profiler.profile] = None
        self._launches0 = 0
        self.trace_file: Optional[str] = None
        self.table_file: Optional[str] = None

    # -- context manager -------------------------------------------------------------------------------------
    def __enter__(self):
        if self.start <= 0:
            self._begin()
        return self

    def __exit__(self, *exc):
        if self._prof is not None:
            self._finish()
        return False

    def step(self):
        self._step += 1
        if self._prof is None and self._step == self.start:
            self._begin()
        elif self._prof is not None and self._step >= self.end:
            self._finish()

    # -- internals --------------------------------------------------------------------------------------------
    def _activities(self):
        acts = []
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        if self.with_cpu or not acts:
            acts.append(torch.profiler.ProfilerActivity.CPU)
        return acts

    def _begin(self):
        from ..ops import loader
        self._launches0 = loader.launch_count() if loader.lib() is not None else 0
        self._prof = torch.profiler.profile(activities=self._activities(), record_shapes=self.record_shapes,
                                            with_stack=self.with_stack, profile_memory=self.with_memory)
        self._prof.__enter__()

    def _finish(self):
        from ..ops import loader
        prof, self._prof = self._prof, None
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        prof.__exit__(None, None, None)
        os.makedirs(self.save_path, exist_ok=True)
        self.trace_file = os.path.join(self.save_path, f"trace_rank{self.rank}_steps{self.start}-{self.end}.json")
        prof.export_chrome_trace(self.trace_file)
        self.table_file = os.path.join(self.save_path, f"kernels_rank{self.rank}_steps{self.start}-{self.end}.txt")
        sort_key = "self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total"
        try:
            table = prof.key_averages().table(sort_by=sort_key, row_limit=60)
        except Exception:  # older/newer attribute names: fall back to the unsorted table
            table = prof.key_averages().table(row_limit=60)
        own = (loader.launch_count() - self._launches0) if loader.lib() is not None else 0
        with open(self.table_file, "w") as f:
            f.write(table)
            f.write(f"\nlaunches of this library's kernels inside the window: {own}\n")


def build_profiler(args) -> StepWindowProfiler:
    """Profiler configured from the ``--profile*`` flags; step numbers count from the first step of this run."""
    return StepWindowProfiler(start=args.profile_step_start, end=args.profile_step_end, save_path=args.profile_save_path,
                              rank=getattr(args, "rank", 0), level=args.profile_level, with_cpu=args.profile_with_cpu,
                              with_stack=args.profile_with_stack, with_memory=args.profile_with_memory,
                              record_shapes=args.profile_record_shapes)
