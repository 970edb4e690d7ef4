"""Turn a profiled training step into the numbers the cost models are fitted on.

Input is what ``utils/profiler.StepWindowProfiler`` writes: a Chrome-trace JSON (``traceEvents`` with ``cat`` = "kernel" /
"gpu_memcpy" events carrying ``name``, ``ts``, ``dur`` in microseconds and the stream in ``tid``).  Kernels are classified
by name into operator classes (GEMM, attention, norm / elementwise, optimizer, and one class per communication kind), and
per class the parser reports call count, total time and - for communication - the time that was NOT hidden under compute on
another stream ("exposed" time: the union of the communication intervals minus their overlap with the union of the compute
intervals), which is what a step actually pays.
reference: mindspeed/auto_settings/module/parse/profiling_parse/* (per-op aggregation of a profiled step; communication
time = total - wait, with a separate overlap figure, tp_comm_perf_predictor.py:53-57).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Sequence, Tuple

CLASSES: Sequence[Tuple[str, str]] = (
    # communication first: fused kernels contain "gemm" in their names too
    ("tp_fused", r"gemm2?_comm|gemm_comm"),
    ("ep_a2a", r"moe_dispatch|moe_combine|all_?to_?all|a2a_strided|SendRecv.*AllToAll"),
    ("dp_reduce", r"dist_opt_fused|ReduceScatter|reduce_scatter"),
    ("dp_gather", r"AllGather|all_gather"),
    ("allreduce", r"AllReduce|all_reduce"),
    ("p2p", r"SendRecv|sendrecv"),
    ("attention", r"flash|fmha|attention|cudnn_generated.*f(prop|ward)|bprop"),
    ("gemm", r"gemm|cutlass|cublas|nvjet|xmma|sm\d+_xmma|ampere_|hopper_"),
    ("optimizer", r"adam|l2norm|clip_coef"),
    ("norm_elementwise", r"rmsnorm|layernorm|layer_norm|rope|swiglu|cross_entropy|softmax|elementwise|vectorized|permute|reduce_kernel"),
    ("memcpy", r"[Mm]emcpy|[Mm]emset"),
)
COMM = ("tp_fused", "ep_a2a", "dp_reduce", "dp_gather", "allreduce", "p2p")


def classify(name: str) -> str:
    for cls, pat in CLASSES:
        if re.search(pat, name):
            return cls
    return "other"


@dataclass
class OpStat:
    calls: int = 0
    total_us: float = 0.0
    exposed_us: float = 0.0
    names: Dict[str, float] = field(default_factory=dict)


@dataclass
class ProfileSummary:
    span_us: float
    busy_us: float
    ops: Dict[str, OpStat]

    def fraction(self, cls: str) -> float:
        return self.ops[cls].total_us / self.busy_us if cls in self.ops and self.busy_us else 0.0

    def table(self) -> str:
        rows = sorted(self.ops.items(), key=lambda kv: -kv[1].total_us)
        out = [f"{'class':18s} {'calls':>7s} {'total ms':>10s} {'exposed ms':>11s} {'share':>6s}"]
        for k, v in rows:
            out.append(f"{k:18s} {v.calls:7d} {v.total_us / 1e3:10.2f} {v.exposed_us / 1e3:11.2f} {v.total_us / max(self.busy_us, 1e-9):6.1%}")
        return "\n".join(out)


def _union(iv: List[Tuple[float, float]]) -> List[Tuple[float, float]]:
    iv = sorted(iv)
    out: List[Tuple[float, float]] = []
    for a, b in iv:
        if out and a <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], b))
        else:
            out.append((a, b))
    return out


def _overlap(a: List[Tuple[float, float]], b: List[Tuple[float, float]]) -> float:
    i = j = 0
    tot = 0.0
    while i < len(a) and j < len(b):
        lo, hi = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if hi > lo:
            tot += hi - lo
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return tot


def summarize(events: Iterable[dict]) -> ProfileSummary:
    ops: Dict[str, OpStat] = {}
    iv: Dict[str, List[Tuple[float, float]]] = {}
    lo, hi = float("inf"), 0.0
    for e in events:
        if e.get("ph") != "X" or e.get("cat") not in ("kernel", "gpu_memcpy", "gpu_memset", "Kernel"):
            continue
        name, ts, dur = e.get("name", ""), float(e.get("ts", 0.0)), float(e.get("dur", 0.0))
        cls = classify(name)
        st = ops.setdefault(cls, OpStat())
        st.calls += 1
        st.total_us += dur
        st.names[name] = st.names.get(name, 0.0) + dur
        iv.setdefault(cls, []).append((ts, ts + dur))
        lo, hi = min(lo, ts), max(hi, ts + dur)
    compute = _union([x for c, v in iv.items() if c not in COMM and c != "memcpy" for x in v])
    for cls in COMM:
        if cls in iv:
            u = _union(iv[cls])
            ops[cls].exposed_us = sum(b - a for a, b in u) - _overlap(u, compute)
    busy = sum(b - a for a, b in _union([x for v in iv.values() for x in v]))
    return ProfileSummary(max(0.0, hi - lo) if hi > lo else 0.0, busy, ops)


def parse_chrome_trace(path: str) -> ProfileSummary:
    with open(path) as f:
        d = json.load(f)
    return summarize(d["traceEvents"] if isinstance(d, dict) else d)


# --- what a search needs to know about a job without running it --------------------------------------------------------
def dump_settings(args, save_path: str) -> str:
    """Write the parsed, validated arguments of this launch (plain values only) to ``<save_path>/auto_settings_args.json``.
    A launcher started with ``OOTB_OPTIMIZER_PARSE_ARGS=TRUE`` does this and exits: the search reads the file instead of
    re-implementing argument parsing (reference: mindspeed/training.py:185-195, auto_settings/module/parse/profiling_parse)."""
    import json
    import os
    os.makedirs(save_path, exist_ok=True)
    plain = {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, list, tuple, type(None))) and not k.startswith("_")}
    out = os.path.join(save_path, "auto_settings_args.json")
    if getattr(args, "rank", 0) == 0:
        with open(out, "w") as f:
            json.dump(plain, f, indent=1, sort_keys=True)
    return out


def dump_model_params(model, pp_rank: int, save_path: str) -> str:
    """Write name, shape, element count and tensor-parallel split of every parameter this pipeline rank holds to
    ``<save_path>/model_params_pp<rank>.json`` (``OOTB_OPTIMIZER_PARSE_MODEL=TRUE``; reference: mindspeed/training.py:273-277).
    One file per pipeline rank, written by the first data- and tensor-parallel rank of the stage."""
    import json
    import os
    os.makedirs(save_path, exist_ok=True)
    rows = []
    for ci, chunk in enumerate(model):
        inner = chunk.module if hasattr(chunk, "module") and not hasattr(chunk, "decoder") else chunk
        for name, p in inner.named_parameters():
            rows.append({"chunk": ci, "name": name, "shape": list(p.shape), "numel": p.numel(), "dtype": str(p.dtype).replace("torch.", ""),
                         "tensor_parallel": bool(getattr(p, "tensor_model_parallel", False)),
                         "partition_dim": int(getattr(p, "partition_dim", -1)), "expert": not getattr(p, "allreduce", True)})
    out = os.path.join(save_path, f"model_params_pp{pp_rank}.json")
    with open(out, "w") as f:
        json.dump({"pp_rank": pp_rank, "parameters": rows, "total_numel": sum(r["numel"] for r in rows)}, f, indent=1)
    return out

