"""Launches short profiling runs of a configuration through ``torch.distributed.run`` child processes and reads back
the measured step time (reference: mindspeed/auto_settings/profile/profiler.py:18-144,
mindspeed/auto_settings/mindspeed_adaptor/mindspeed_executor.py)."""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
from typing import List, Optional

from .search_space import SearchConfig

_TIME_RE = re.compile(r"elapsed time per iteration \(ms\): ([0-9.]+)")


class TorchrunExecutor:
    def __init__(self, base_flags: List[str], nproc: int, script: Optional[str] = None, iters: int = 4, master_port: int = 29650,
                 timeout_s: int = 900, env: Optional[dict] = None, profile_dir: Optional[str] = None):
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        self.script = script or os.path.join(root, "pretrain_gpt.py")
        self.base_flags, self.nproc, self.iters, self.port, self.timeout_s = list(base_flags), nproc, iters, master_port, timeout_s
        self.env = env or {}
        # with a profile directory every measured run also records one step (rank 0) as a Chrome trace; ``last_trace`` is
        # the file of the most recent run, for profiling_parse / cost_model.learn_from_profile
        self.profile_dir, self.last_trace, self._runs = profile_dir, None, 0
        self.traces: List[tuple] = []            # (configuration, trace file) of every successful profiled run

    def command(self, cfg: SearchConfig) -> List[str]:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(self.nproc),
                "--master-addr", "127.0.0.1", "--master-port", str(self.port), self.script] + self.base_flags + cfg.to_flags() + \
               ["--train-iters", str(self.iters), "--log-interval", "1"] + self._profile_flags()

    def _profile_flags(self) -> List[str]:
        if not self.profile_dir:
            return []
        d = os.path.join(self.profile_dir, f"run{self._runs}")
        return ["--profile", "--profile-step-start", str(max(1, self.iters - 2)), "--profile-step-end", str(max(2, self.iters - 1)),
                "--profile-ranks", "0", "--profile-save-path", d]

    def _find_trace(self) -> Optional[str]:
        d = os.path.join(self.profile_dir, f"run{self._runs}")
        for root, _, files in os.walk(d):
            for f in files:
                if f.endswith(".json"):
                    return os.path.join(root, f)
        return None

    def __call__(self, cfg: SearchConfig) -> Optional[float]:
        env = dict(os.environ, **self.env)
        try:
            r = subprocess.run(self.command(cfg), capture_output=True, text=True, timeout=self.timeout_s, env=env)
        except subprocess.TimeoutExpired:
            return None
        if self.profile_dir:
            self.last_trace = self._find_trace() if r.returncode == 0 else None
            if self.last_trace:
                self.traces.append((cfg, self.last_trace))
            self._runs += 1
        if r.returncode != 0:
            return None
        times = [float(x) for x in _TIME_RE.findall(r.stdout)]
        if len(times) < 2:
            return None
        steady = times[1:]
        return sum(steady) / len(steady)
