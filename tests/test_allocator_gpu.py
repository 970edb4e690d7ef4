"""Device build of the native caching allocator as torch's CUDA allocator, and the pinned-host swap pool."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code: str):
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def test_training_step_on_native_allocator():
    out = _run("""
        import torch
        from mindspeed_b200.memory import allocator as A
        assert A.install(), "allocator must install before the first CUDA allocation"
        A.enable_trace(1 << 16)
        A.set_tags(0, 0)
        dev = torch.device("cuda", 0)
        net = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.GELU(), torch.nn.Linear(4096, 1024)).to(dev)
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
        x = torch.randn(2048, 1024, device=dev)
        losses = []
        for step in range(3):
            A.set_tags(step, 0)
            loss = net(x).pow(2).mean()
            A.set_tags(step, 1)
            loss.backward()
            opt.step(); opt.zero_grad()
            losses.append(float(loss))
        torch.cuda.synchronize()
        s = A.device_stats()
        assert s["num_mallocs"] > 10 and s["allocated_bytes"] > 0 and s["reserved_bytes"] >= s["allocated_bytes"], s
        assert s["num_segment_allocs"] < s["num_mallocs"], "blocks must be reused from the cache"
        assert losses[2] < losses[0]
        ev = A.read_trace()
        assert any(e["phase"] == 1 for e in ev) and any(e["is_free"] for e in ev)
        # soft limit + pressure callback: the callback drops a big tensor so the next allocation fits
        held = [torch.empty(256 << 20, dtype=torch.uint8, device=dev)]
        A.empty_cache()            # otherwise the allocator makes room by returning cached segments first
        A.set_limit(A.device_stats()["reserved_bytes"] + (64 << 20))
        calls = []
        def on_pressure(need, d):
            calls.append(need)
            held.clear()
            return 256 << 20
        A.set_pressure_callback(on_pressure)
        y = torch.empty(200 << 20, dtype=torch.uint8, device=dev)
        assert calls and y.numel() == 200 << 20
        A.set_pressure_callback(None)
        A.set_limit(0)
        print("OK", s["num_mallocs"], s["num_segment_allocs"])
    """)
    assert "OK" in out


def test_swap_pool_roundtrip():
    out = _run("""
        import ctypes, torch
        from mindspeed_b200.ops import loader
        L = loader.require_lib()
        L.msb_swap_pinned_bytes.restype = ctypes.c_ulonglong
        x = torch.randn(8 << 20, device="cuda")
        ref = x.clone()
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        slot = L.msb_swap_out(ctypes.c_void_p(x.data_ptr()), ctypes.c_ulonglong(x.numel() * 4), st)
        assert slot >= 0, loader.last_error() if hasattr(loader, "last_error") else slot
        assert L.msb_swap_wait(slot) == 0
        x.zero_()
        assert L.msb_swap_in(slot, ctypes.c_void_p(x.data_ptr()), ctypes.c_ulonglong(x.numel() * 4), st, 1) == 0
        torch.cuda.synchronize()
        assert torch.equal(x, ref)
        assert L.msb_swap_pinned_bytes() >= x.numel() * 4
        print("OK")
    """)
    assert "OK" in out
