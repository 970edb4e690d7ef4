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


def test_plan_steps_fits_the_wall_clock_budget():
    sys.path.insert(0, ROOT)
    import bench
    # 29.5 s steps, 480 s left, driver asks for 20 steps: the timed loop is cut, e2e and baseline keep two steps each
    k, ke, kb, trunc = bench.plan_steps(29.5, 480.0, 20, -1, -1)
    assert trunc and ke == 2 and kb == 2 and k >= 2
    assert (k + ke + kb + 1) * 29.5 <= 480.0
    # short steps: everything fits, nothing is cut
    k, ke, kb, trunc = bench.plan_steps(0.7, 500.0, 20, -1, -1)
    assert (k, trunc) == (20, False) and ke == 5 and kb == 5
    # almost no time left: the baseline arm goes first, then e2e shrinks, the timed loop keeps two steps
    k, ke, kb, trunc = bench.plan_steps(30.0, 120.0, 20, -1, -1)
    assert k == 2 and kb == 0 and ke == 1 and trunc
    # explicit requests are honoured
    assert bench.plan_steps(1.0, 1000.0, 3, 0, 0) == (3, 0, 0, False)


def test_layout_args_per_model():
    sys.path.insert(0, ROOT)
    import bench
    a = bench.parse(["--gpus", "8"])
    lay, par, rl = bench.layout_args(a, 8)
    assert par == "tp8+sp+distopt" and rl == 0 and "--use-fused-tp-comm" in lay and "--reuse-fp32-param" not in lay
    lay, par, rl = bench.layout_args(a, 1)
    assert par == "tp1+distopt" and rl == 8 and "--reuse-fp32-param" in lay
    a = bench.parse(["--gpus", "8", "--model", "mixtral-8x7b"])
    lay, par, rl = bench.layout_args(a, 8)
    assert "--expert-model-parallel-size" in lay and par.startswith("ep8")
    a = bench.parse(["--gpus", "8", "--model", "llama2-13b"])
    lay, par, rl = bench.layout_args(a, 8)
    assert par == "cp4xtp2+sp+distopt" and rl == 40
