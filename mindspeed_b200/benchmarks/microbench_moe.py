"""Multi-GPU micro-benchmark of MoE token dispatch + combine: peer-memory kernels against NCCL all-to-all-v.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m mindspeed_b200.benchmarks.microbench_moe [--tokens 4096] [--hidden 4096] [--experts 8] [--topk 2] [--json out.json]

Every rank routes ``tokens`` rows of width ``hidden`` (bf16) to ``topk`` of ``experts`` experts spread over the N ranks
(uniform random routing, fixed seed).  Timed per rank with CUDA events (3 warm-up rounds, L2 flushed and a barrier
before each timed round, short device-side delay so host launch latency is outside the interval), maximum over ranks
of the median:
    dispatch   token_permutation   (library: permute + all-to-all-v tokens + all-to-all-v probabilities + chunk sort)
    combine    token_unpermutation (library: chunk sort + all-to-all-v + un-permute)
The routing pre-processing (count exchange and the host read of the split sizes) is common to both paths and is
inside the dispatch interval of both.  Roofline: bytes that must leave / enter a GPU over NVLink at 770 GB/s,
i.e. tokens * topk * (N-1)/N * hidden * 2 bytes per direction.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import torch.nn.functional as F
    from ..config import TransformerConfig
    from ..parallel import parallel_state as ps
    from ..parallel.moe.fused_dispatcher import FusedAlltoAllTokenDispatcher
    from ..parallel.moe.token_dispatcher import MoEAlltoAllTokenDispatcher
    from ..ops import gemm as G
    from ..ops import loader
    ps.initialize_model_parallel(expert_model_parallel_size=world)
    L = loader.require_lib()
    cfg = TransformerConfig(num_layers=1, hidden_size=a.hidden, num_attention_heads=8, ffn_hidden_size=a.hidden, num_moe_experts=a.experts,
                            moe_router_topk=a.topk, moe_grouped_gemm=True, gated_linear_unit=True, activation_func=F.silu,
                            add_bias_linear=False, expert_model_parallel_size=world, moe_token_dispatcher_type="alltoall",
                            optimization_level=2, params_dtype=torch.bfloat16, bf16=True)
    e_loc = a.experts // world
    idx = list(range(rank * e_loc, (rank + 1) * e_loc))
    lib = MoEAlltoAllTokenDispatcher(e_loc, idx, cfg)
    fus = FusedAlltoAllTokenDispatcher(e_loc, idx, cfg)
    g = torch.Generator(device="cuda").manual_seed(99 + rank)
    x = (torch.randn(a.tokens, 1, a.hidden, device="cuda", generator=g) * 0.1).bfloat16()
    scores = torch.rand(a.tokens, a.experts, device="cuda", generator=g)
    topv, topi = scores.topk(a.topk, dim=1)
    rmap = torch.zeros_like(scores, dtype=torch.bool).scatter(1, topi, True)
    probs = torch.zeros_like(scores).scatter(1, topi, torch.softmax(topv, dim=1)).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters=8, warmup=3):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            L.msb_l2_flush(ctypes.c_void_p(flush.data_ptr()), ctypes.c_size_t(flush.numel()), ctypes.c_void_p(loader.stream_ptr()))
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(1_000_000)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.median(ts)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {}
    with torch.no_grad():
        for name, d in (("library", lib), ("fused", fus)):
            rows, tpe, rp = d.token_permutation(x, probs, rmap)
            y = rows * 1.0
            out, _ = d.token_unpermutation(y)
            res[name + "_out"] = out
            res[name + "_dispatch_ms"] = timed(lambda: d.token_permutation(x, probs, rmap))
            d.token_permutation(x, probs, rmap)
            res[name + "_combine_ms"] = timed(lambda: d.token_unpermutation(y))
        torch.cuda.synchronize()
        G.check_status()
    diff = (res["library_out"].float() - res["fused_out"].float()).abs().max().item()
    ref = res["library_out"].float().abs().max().item()
    link_bytes = a.tokens * a.topk * (world - 1) / world * a.hidden * 2
    roof = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    if rank == 0:
        for phase in ("dispatch", "combine"):
            f, l = res[f"fused_{phase}_ms"], res[f"library_{phase}_ms"]
            print(f"{phase:9s} tokens={a.tokens} hidden={a.hidden} experts={a.experts} topk={a.topk} ep={world}: fused {f:7.3f} ms  "
                  f"library {l:7.3f} ms  roofline {roof:6.3f} ms  fused {roof / f:4.2f} / library {roof / l:4.2f} of roofline  "
                  f"speedup {l / f:4.2f}x", flush=True)
        print(f"max |fused - library| = {diff:.3g} (output range {ref:.3g}); fused calls {fus.fused_calls}, fallbacks {fus.fallback_calls}")
        if a.json:
            os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
            with open(a.json, "w") as f:
                json.dump({k: v for k, v in res.items() if not k.endswith("_out")} | {"roofline_ms": roof, "world": world, "args": vars(a),
                          "max_abs_diff": diff}, f, indent=1)
    dist.barrier()
    from ..parallel.symm_mem import destroy_heaps
    destroy_heaps()
    ps.destroy_model_parallel()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
