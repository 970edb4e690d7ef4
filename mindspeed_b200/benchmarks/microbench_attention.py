"""Attention micro-benchmark: tcgen05 forward / backward vs the framework library (part of ``benchmarks.microbench``)."""
import torch

from ..training.flops import measured_peaks
from .microbench import time_fn


def bench_attention(out):
    from ..ops.flash_sm100_impl import flash_bwd, flash_fwd
    pk = measured_peaks()
    for (s, nq, nkv) in [(8192, 32, 8), (8192, 4, 1), (4096, 32, 8), (16384, 8, 2)]:
        q = torch.randn(s, 1, nq, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(s, 1, nkv, 128, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(s, 1, nkv, 128, device="cuda", dtype=torch.bfloat16)
        do = torch.randn(s, 1, nq, 128, device="cuda", dtype=torch.bfloat16)
        fl = 4.0 * s * s * nq * 128 / 2
        rows = {}
        rows["fwd_ours"] = (time_fn(lambda: flash_fwd(q, k, v, True, 128 ** -0.5)), fl)
        rows["fwd_ours_single_tile"] = (time_fn(lambda: flash_fwd(q, k, v, True, 128 ** -0.5, kernel=1)), fl)
        qb, kb, vb = q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3)
        rows["fwd_library"] = (time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, is_causal=True, enable_gqa=True)), fl)
        o, lse = flash_fwd(q, k, v, True, 128 ** -0.5)
        rows["bwd_ours"] = (time_fn(lambda: flash_bwd(do, q, k, v, o, lse, True, 128 ** -0.5)), 2.5 * fl)
        ql, kl, vl = (t.detach().clone().requires_grad_(True) for t in (qb, kb, vb))
        ol = torch.nn.functional.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=True)
        dol = do.permute(1, 2, 0, 3)
        rows["bwd_library"] = (time_fn(lambda: torch.autograd.grad(ol, (ql, kl, vl), dol, retain_graph=True)), 2.5 * fl)
        for name, (t, f) in rows.items():
            tf = f / t / 1e9
            out.append({"op": f"flash/s{s}_h{nq}_{name}", "ms": t, "tflops": tf, "frac_of_measured_bf16_peak": tf / pk["bf16_tflops"]})
            print(f"flash s={s} heads={nq}/{nkv} {name:22s} {t:8.3f} ms {tf:8.1f} TFLOP/s  {tf / pk['bf16_tflops']:.2f} of {pk['source']} peak", flush=True)
