"""bench.py contract pieces that need no GPU: the reference arm's line and the clock-sample parser."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "3"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "torch_npu" in d["unavailable"]


def test_clock_sampler_parses_and_flags_reasons():
    sys.path.insert(0, ROOT)
    import bench
    s = bench.ClockSampler(0)
    s.proc = object()
    s.lines = ["1965, 1965, 120.5, Not Active, Not Active, Not Active, Not Active",
               "1410, 1965, 995.1, Not Active, Not Active, Not Active, Active",
               "1395, 1965, 990.0, Not Active, Not Active, Not Active, Active",
               "garbage"]
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0, "kill": lambda self: None})()
    out = s.stop()
    assert out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"] and out["samples"] == 3
    assert 1390 <= out["sm_mhz"] <= 1415          # median of the samples under load, not of the idle one
