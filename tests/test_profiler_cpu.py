"""Step-window profiler: records only inside the window and leaves a trace plus a kernel table."""
import os

import torch

from mindspeed_b200.utils.profiler import StepWindowProfiler


def test_window_and_outputs(tmp_path):
    p = StepWindowProfiler(start=2, end=4, save_path=str(tmp_path), rank=3, level="level1")
    x = torch.randn(64, 64)
    with p:
        for i in range(6):
            (x @ x).sum().item()
            p.step()
            if i == 0:
                assert p._prof is None          # step 1 done, window opens after step 2
            if i == 2:
                assert p._prof is not None      # inside the window
    assert p._prof is None
    assert p.trace_file and os.path.getsize(p.trace_file) > 0
    txt = open(p.table_file).read()
    assert "launches of this library's kernels inside the window" in txt
    assert "rank3" in os.path.basename(p.trace_file)
