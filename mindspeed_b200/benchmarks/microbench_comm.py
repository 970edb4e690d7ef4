"""Multi-GPU micro-benchmark of the fused GEMM + collective kernels against the library path.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m mindspeed_b200.benchmarks.microbench_comm [--json out.json] [--seq 8192]

For each tensor-parallel linear of a Llama-3-8B-shape layer at TP = N it times, on every rank,

  fused   : one launch of the all-gather->GEMM kernel, or the GEMM->reduce-scatter kernel plus its owner-side sum
  library : NCCL all_gather_into_tensor + cuBLAS GEMM, or cuBLAS GEMM + NCCL reduce_scatter_tensor

with CUDA events on the launching stream: 3 warm-up launches, then 10 x (256 MB buffer rewritten so that operands start
outside L2, one call) back to back after a barrier and a device-side delay that lets the host queue the loop, minus the
same loop with the rewrite alone; median of 3 such measurements, maximum over ranks.  The roofline for a fused kernel is the slower of

  FLOPs / measured cuBLAS bf16 peak           and           bytes that must cross NVLink per GPU / 770 GB/s

(770 GB/s is the measured per-direction peer-copy bandwidth of one GPU through NVSwitch); the printed fraction is
roofline time / achieved time.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _timed(fn, group, flush_buf, L, loader, iters=10, warmup=3):
    """Steady-state time of one call: ``iters`` x (L2 flush + call) back to back between two events, minus the same loop
    with the flush alone.  A device-side delay in front of the first event lets the host queue the whole loop first, so
    the interval is device execution; ranks start together after a barrier and stay together through the collective
    itself, so start-up skew is paid once per loop, not once per call."""
    for _ in range(warmup):
        fn()

    def loop(with_fn):
        torch.cuda.synchronize()
        dist.barrier(group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(12_000_000)
        e0.record()
        for _ in range(iters):
            L.msb_l2_flush(ctypes.c_void_p(flush_buf.data_ptr()), ctypes.c_size_t(flush_buf.numel()),
                           ctypes.c_void_p(loader.stream_ptr()))
            if with_fn:
                fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ts = sorted(loop(True) - loop(False) for _ in range(3))
    t = torch.tensor([ts[1]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--json", default=None)
    p.add_argument("--seq", type=int, default=8192)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--ffn", type=int, default=14336)
    p.add_argument("--qkv", type=int, default=6144)
    p.add_argument("--timeline", action="store_true", help="print CTA 0's in-kernel time stamps of one fused launch per case")
    a = p.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    group = dist.group.WORLD
    from ..ops import loader
    from ..ops.fused_comm import FusedOps
    from ..parallel.comm_ops import DefaultOps
    from ..training.flops import measured_peaks
    L = loader.require_lib()
    pk = measured_peaks()
    peak = pk["bf16_tflops"] * 1e12
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    S, H, F, Q = a.seq, a.hidden, a.ffn, a.qkv
    n = world
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def rnd(*shape):
        return (torch.randn(*shape, device="cuda", dtype=torch.bfloat16, generator=g) * 0.05)

    cases = [
        # name, kind, local x, weight, nt
        ("qkv  ag->gemm fwd", "ag", rnd(S // n, H), rnd(Q // n, H), True),
        ("fc1  ag->gemm fwd", "ag", rnd(S // n, H), rnd(2 * F // n, H), True),
        ("proj gemm->rs fwd", "rs", rnd(S, H // n), rnd(H, H // n), True),
        ("fc2  gemm->rs fwd", "rs", rnd(S, F // n), rnd(H, F // n), True),
        # backward of a column linear: dgrad = dy @ W followed by reduce-scatter
        ("qkv  gemm->rs dgrad", "rs", rnd(S, Q // n), rnd(Q // n, H), False),
        ("fc1  gemm->rs dgrad", "rs", rnd(S, 2 * F // n), rnd(2 * F // n, H), False),
        # backward of a row linear: dgrad = allgather(dy) @ W
        ("proj ag->gemm dgrad", "ag", rnd(S // n, H), rnd(H, H // n), False),
        ("fc2  ag->gemm dgrad", "ag", rnd(S // n, H), rnd(H, F // n), False),
    ]
    results = []
    for name, kind, x, w, nt in cases:
        if kind == "ag":
            m, k = x.shape[0] * n, x.shape[1]
            nout = w.shape[0] if nt else w.shape[1]
            link_bytes = (n - 1) / n * m * k * 2
            fused = lambda: FusedOps.allgather_matmul(x, w, group, nt)
            lib = lambda: DefaultOps.allgather_matmul(x, w, group, nt)
        else:
            m, k = x.shape
            nout = w.shape[0] if nt else w.shape[1]
            link_bytes = (n - 1) / n * m * nout * 2
            fused = lambda: FusedOps.matmul_reduce_scatter(x, w, group, nt)
            lib = lambda: DefaultOps.matmul_reduce_scatter(x, w, group, nt)
        flops = 2.0 * m * nout * k
        # numerics first: both paths must agree within bf16 rounding of a k-term sum
        yf = fused()
        yl = lib()
        yf = yf[0] if isinstance(yf, tuple) else yf
        yl = yl[0] if isinstance(yl, tuple) else yl
        err = (yf.float() - yl.float()).abs().max().item()
        ref = yl.float().abs().max().item()
        if a.timeline:
            from ..ops import fused_comm as FC
            FC.TIMELINE = torch.zeros(8, dtype=torch.int64, device="cuda")
            torch.cuda.synchronize(); dist.barrier(group); fused(); torch.cuda.synchronize()
            ts = FC.TIMELINE.tolist()
            FC.TIMELINE = None
            if rank == 0:
                rel = [(t - ts[0]) / 1e3 if t else None for t in ts]
                print(f"    timeline us (CTA 0): handshake {rel[1]}, copy done {rel[2]}, loads issued {rel[3]}, epilogue done {rel[4]}, "
                      f"rs flags in {rel[5]}, end {rel[6]}", flush=True)
        t_f = _timed(fused, group, flush, L, loader)
        t_l = _timed(lib, group, flush, L, loader)
        t_roof = max(flops / peak, link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        row = {"case": name, "M": m, "N": nout, "K": k, "world": n, "fused_ms": t_f, "library_ms": t_l,
               "roofline_ms": t_roof, "fused_frac_of_roofline": t_roof / t_f, "library_frac_of_roofline": t_roof / t_l,
               "bound": "gemm" if flops / peak > link_bytes / (NVLINK_GBS * 1e9) else "nvlink",
               "max_abs_diff": err, "max_abs_ref": ref}
        results.append(row)
        if rank == 0:
            print(f"{name:22s} M={m:5d} N={nout:5d} K={k:5d}  fused {t_f:7.3f} ms  library {t_l:7.3f} ms  roofline {t_roof:6.3f} ms "
                  f"({row['bound']})  fused {t_roof / t_f:4.2f} / library {t_roof / t_l:4.2f} of roofline  maxdiff {err:.3g}/{ref:.3g}",
                  flush=True)
    if rank == 0 and a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        with open(a.json, "w") as f:
            json.dump({"peaks": pk, "nvlink_gbs": NVLINK_GBS, "world": n, "results": results}, f, indent=1)
    dist.barrier()
    from ..parallel.symm_mem import destroy_heaps
    destroy_heaps()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
