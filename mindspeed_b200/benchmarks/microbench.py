"""Kernel micro-benchmarks with roofline fractions.

  python -m mindspeed_b200.benchmarks.microbench [gemm|fp8|elementwise|attention|all] [--json out.json]

Timing: CUDA events on the launching stream, >= 3 warm-up launches, L2 flushed (a 256 MB buffer is rewritten)
between timed launches, median of the timed launches.  Fractions are relative to the measured copy bandwidth
and cuBLAS bf16 throughput recorded in MEASURED_PEAKS.json when present (nominal figures otherwise).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import statistics
import sys

import torch

from ..ops import loader
from ..training.flops import measured_peaks


def _flush_buf():
    if not hasattr(_flush_buf, "b"):
        _flush_buf.b = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    return _flush_buf.b


def time_fn(fn, iters=10, warmup=3, flush=True):
    L = loader.require_lib()
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        # a device-side delay first: the host enqueues the flush, the start event and fn's launches while the GPU spins, so
        # the interval between the events holds device time only, not the host's launch latency (which would otherwise add
        # 50-100 us to every kernel shorter than that)
        torch.cuda._sleep(400000)
        if flush:
            b = _flush_buf()
            L.msb_l2_flush(ctypes.c_void_p(b.data_ptr()), ctypes.c_size_t(b.numel()), ctypes.c_void_p(loader.stream_ptr()))
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def bench_gemm(out, variants=False):
    from ..ops import gemm as G
    pk = measured_peaks()
    shapes = [("qkv_fwd_tp1", 8192, 6144, 4096), ("fc1_fwd_tp1", 8192, 28672, 4096), ("fc2_fwd_tp1", 8192, 4096, 14336),
              ("proj_fwd_tp1", 8192, 4096, 4096), ("qkv_fwd_tp8", 8192, 768, 4096), ("fc1_fwd_tp8", 8192, 3584, 4096),
              ("fc2_fwd_tp8", 8192, 4096, 1792), ("proj_fwd_tp8", 8192, 4096, 512), ("square_8k", 8192, 8192, 8192)]
    for name, M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        fl = 2.0 * M * N * K
        rows = {}
        if variants:      # every kernel variant side by side (1 = one-CTA, 2 / 3 = CTA pair 256x256 / 256x128)
            for v in (1, 2, 3):
                with G.variant(v):
                    rows[f"fwd_v{v}"] = time_fn(lambda: G.linear_fwd(x, w))
                    rows[f"dgrad_v{v}"] = time_fn(lambda: G.linear_dgrad(dy, w))
                    rows[f"wgrad_v{v}"] = time_fn(lambda: G.linear_wgrad(dy, x, acc))
        rows["fwd_ours"] = time_fn(lambda: G.linear_fwd(x, w))
        rows["fwd_cublas"] = time_fn(lambda: torch.matmul(x, w.t()))
        rows["dgrad_ours"] = time_fn(lambda: G.linear_dgrad(dy, w))
        rows["dgrad_cublas"] = time_fn(lambda: torch.matmul(dy, w))
        rows["wgrad_ours"] = time_fn(lambda: G.linear_wgrad(dy, x, acc))
        rows["wgrad_cublas"] = time_fn(lambda: torch.matmul(dy.t(), x))
        G.check_status()
        for k, ms in rows.items():
            tf = fl / ms / 1e9
            out.append({"op": f"gemm/{name}/{k}", "M": M, "N": N, "K": K, "ms": ms, "tflops": tf,
                        "frac_of_measured_bf16_peak": tf / pk["bf16_tflops"]})
            print(f"{name:14s} {k:13s} {ms:8.3f} ms {tf:8.1f} TFLOP/s  {tf / pk['bf16_tflops']:.2f} of {pk['source']} peak", flush=True)


def bench_elementwise(out):
    from ..ops.activation import swiglu
    from ..ops.norm import rms_norm
    from ..ops.rope import rope_packed_qkv_
    from ..ops.adam import adam_flat
    pk = measured_peaks()
    rows, h = 8192, 4096

    def rec(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        out.append({"op": name, "ms": ms, "GBps": gbs, "frac_of_measured_copy_bw": gbs / pk["hbm_gbs"]})
        print(f"{name:28s} {ms:8.3f} ms {gbs:8.0f} GB/s  {gbs / pk['hbm_gbs']:.2f} of {pk['source']} copy bandwidth", flush=True)

    x = torch.randn(4 * rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    rec("rmsnorm_fwd", time_fn(lambda: rms_norm(x, w)), 2 * x.numel() * 2)
    y = rms_norm(x, w)
    g = torch.randn_like(y)
    rec("rmsnorm_bwd", time_fn(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True)), 3 * x.numel() * 2)
    from ..ops.norm import add_rms_norm
    r = torch.randn_like(x, requires_grad=True)
    rec("add_rmsnorm_fwd", time_fn(lambda: add_rms_norm(x, r, w)), 4 * x.numel() * 2)
    hh, yy = add_rms_norm(x, r, w)
    g2 = torch.randn_like(hh)
    rec("add_rmsnorm_bwd", time_fn(lambda: torch.autograd.grad((hh, yy), (x, r, w), (g2, g), retain_graph=True)), 4 * x.numel() * 2)
    del r, hh, yy, g2
    f = 14336
    z = torch.randn(rows, 2 * f, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    rec("swiglu_fwd", time_fn(lambda: swiglu(z)), 3 * rows * f * 2)
    zz = swiglu(z)
    gz = torch.randn_like(zz)
    rec("swiglu_bwd", time_fn(lambda: torch.autograd.grad(zz, z, gz, retain_graph=True)), 5 * rows * f * 2)
    qkv = torch.randn(rows, 1, 6144, device="cuda", dtype=torch.bfloat16)
    cos = torch.randn(rows, 128, device="cuda"); sin = torch.randn(rows, 128, device="cuda")
    rec("rope_packed_qkv", time_fn(lambda: rope_packed_qkv_(qkv, cos, sin, 8, 4, 128)), 2 * rows * 5120 * 2)
    n = 256 * 1024 * 1024
    p = torch.randn(n, device="cuda"); gg = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rec("adam_flat", time_fn(lambda: adam_flat(p, gg, m, v, p16, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1), iters=5), n * (4 * 4 + 3 * 4 + 2))


def bench_fp8(out):
    """Block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales) on the layer shapes; fractions are of the
    measured *bf16* cuBLAS peak (no fp8 library figure is recorded), so 1.0 means parity with bf16 at half the bytes."""
    from ..ops import gemm_fp8 as F
    from ..ops.quant import quant_128x128, quant_1x128
    pk = measured_peaks()
    for name, M, N, K in (("fc1_fwd_tp1", 8192, 28672, 4096), ("fc2_fwd_tp1", 8192, 4096, 14336), ("fc1_fwd_tp8", 8192, 3584, 4096),
                          ("expert_fc1", 16384, 3072, 4096), ("square_8k", 8192, 8192, 8192)):
        xq, xs = quant_1x128(torch.randn(M, K, device="cuda"))
        wq, ws = quant_128x128(torch.randn(N, K, device="cuda") * 0.05)
        ms = time_fn(lambda: F.fp8_gemm(xq, xs, wq, ws))
        tf = 2.0 * M * N * K / ms / 1e9
        out.append({"kernel": "gemm_fp8_blockscaled", "case": name, "ms": ms, "tflops": tf, "frac_of_bf16_peak": tf / pk["bf16_tflops"]})
        print(f"{name:14s} fp8_blockscaled  {ms:8.3f} ms  {tf:8.1f} TFLOP/s  {tf / pk['bf16_tflops']:.2f} of measured bf16 peak", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="?", default="all")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    out = []
    if a.what in ("gemm", "gemm_variants", "all"):
        bench_gemm(out, variants=(a.what == "gemm_variants"))
    if a.what in ("fp8", "all"):
        bench_fp8(out)
    if a.what in ("elementwise", "all"):
        bench_elementwise(out)
    if a.what in ("attention", "all"):
        try:
            from .microbench_attention import bench_attention
            bench_attention(out)
        except ImportError:
            pass
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"peaks": measured_peaks(), "results": out}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
