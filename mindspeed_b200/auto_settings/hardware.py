"""Hardware description used by the cost models: measured on the box where possible.

The reference keys its communication model on a table of interconnect domain sizes
(mindspeed/auto_settings/module/communication/comm_hardware/comm_hardware_info.py:7-40).  One NVSwitch domain gives every
GPU the same bandwidth to every peer, so the table collapses to a few measured numbers: dense bf16 GEMM throughput, HBM
copy bandwidth, NVLink per-direction bandwidth and all-reduce bus bandwidth.  ``probe()`` measures GEMM and copy on the
current GPU; the NVLink figures come from a multi-rank probe (``probe_collectives``) or the defaults recorded for this
machine class."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict


@dataclass
class Hardware:
    bf16_tflops: float = 1413.5          # sustained dense bf16 (cuBLAS, measured on B200)
    hbm_gbs: float = 6540.0              # measured copy bandwidth
    hbm_gib: float = 178.0               # usable device memory
    nvlink_gbs: float = 770.0            # measured peer copy, per direction per GPU
    allreduce_bus_gbs: float = 725.0     # measured 8-rank all-reduce bus bandwidth at 1 GiB
    collective_latency_us: float = 12.0
    p2p_latency_us: float = 6.0
    gpus_per_node: int = 8
    internode_gbs: float = 50.0          # per GPU, when a job spans nodes (400 Gb/s NIC)

    @staticmethod
    def load(path=None):
        hw = Hardware()
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        p = path or os.path.join(root, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            try:
                with open(p) as f:
                    d = json.load(f)
                hw.bf16_tflops = d.get("bf16_tflops_sustained", hw.bf16_tflops)
                hw.hbm_gbs = d.get("hbm_gbs", hw.hbm_gbs)
                for k in ("nvlink_gbs", "allreduce_bus_gbs"):
                    if k in d:
                        setattr(hw, k, d[k])
            except Exception:
                pass
        return hw

    def save(self, path):
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=1)


def probe(hw: Hardware = None) -> Hardware:
    """Measure GEMM throughput and copy bandwidth on the current GPU (CUDA events, warm-up, best of 5)."""
    import torch
    hw = hw or Hardware.load()
    if not torch.cuda.is_available():
        return hw
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    src = torch.empty(1 << 29, device="cuda", dtype=torch.bfloat16)
    dst = torch.empty_like(src)

    def best(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return min(ts)

    hw.bf16_tflops = 2 * 8192 ** 3 / best(lambda: a @ b) / 1e9
    hw.hbm_gbs = 2 * src.numel() * 2 / best(lambda: dst.copy_(src)) / 1e6
    return hw


def probe_collectives(hw: Hardware, group=None, nbytes=1 << 28) -> Hardware:
    """All-reduce bus bandwidth of ``group`` (call on every rank; device-timed, max over ranks)."""
    import torch
    import torch.distributed as dist
    if not (torch.cuda.is_available() and dist.is_initialized()):
        return hw
    n = dist.get_world_size(group)
    x = torch.empty(nbytes // 2, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        dist.all_reduce(x, group=group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(); e0.record()
    for _ in range(5):
        dist.all_reduce(x, group=group)
    e1.record(); torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / 5], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
    hw.allreduce_bus_gbs = nbytes * 2 * (n - 1) / n / ms.item() / 1e6
    return hw
