"""Training-loop integration of the memory managers and QAT flags: same losses as the plain run (the policies only
change where activations live / whether they are recomputed), QAT stays close."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402
from test_pipeline_cpu import _train  # noqa: E402


@pytest.mark.parametrize("extra,exact", [
    (["--adaptive-recompute-device-size", "1", "--adaptive-recompute-profiling-step", "1"], True),
    (["--adaptive-recompute-device-swap", "--adaptive-recompute-device-size", "1", "--adaptive-recompute-profiling-step", "2"], True),
    (["--adaptive-memory-optimization", "--adaptive-recompute-device-size", "1", "--adaptive-recompute-profiling-step", "1"], True),
    (["--smart-swap"], True),
    (["--qat-scheme", "w8a16"], False),
])
def test_flag_runs_and_matches_plain_training(extra, exact):
    from test_pipeline_cpu import _reference_losses
    ref = _reference_losses(())
    got = run_distributed(_train, 1, extra, False)[0]
    for a, b in zip(ref, got):
        tol = 2e-4 if exact else 2e-2
        assert abs(a - b) < tol * max(1.0, abs(a)), (ref, got)
