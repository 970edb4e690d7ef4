"""Small, self-terminating workloads for Nsight Compute captures of single kernels.

  python -m mindspeed_b200.benchmarks.ncu_targets gemm        # 3 launches each of fwd / dgrad / wgrad, 8192^3 bf16
  python -m mindspeed_b200.benchmarks.ncu_targets elementwise # rmsnorm / swiglu / rope / adam / cross-entropy once each
  python -m mindspeed_b200.benchmarks.ncu_targets fp8         # 3 launches of the block-scaled fp8 GEMM, 8192 x 8192 x 8192
  python -m mindspeed_b200.benchmarks.ncu_targets gemm_tp8    # the four forward GEMM shapes of a Llama-3-8B layer at TP8
  python -m mindspeed_b200.benchmarks.ncu_targets flash       # 2 launches each of flash-attention forward and backward

Inputs exceed the 126 MB L2 but stay well under 2 GB on the device; there are only a handful of launches, so a
``--set full`` capture ends by itself within a minute or two.
"""
import sys

import torch


def gemm():
    from ..ops import gemm as G
    M = N = K = 8192
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    for _ in range(3):
        G.linear_fwd(x, w)
        G.linear_dgrad(dy, w)
        G.linear_wgrad(dy, x, acc)
    torch.cuda.synchronize()
    G.check_status()


def elementwise():
    from ..ops.activation import swiglu
    from ..ops.adam import adam_flat
    from ..ops.cross_entropy import fused_vocab_parallel_cross_entropy
    from ..ops.norm import rms_norm
    from ..ops.rope import rope_packed_qkv_
    rows, h = 16384, 4096
    x = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = rms_norm(x, w)
    y.backward(torch.randn_like(y))
    z = torch.randn(8192, 2 * 14336, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    s = swiglu(z)
    s.backward(torch.randn_like(s))
    qkv = torch.randn(8192, 1, 6144, device="cuda", dtype=torch.bfloat16)
    cs = torch.randn(8192, 128, device="cuda")
    rope_packed_qkv_(qkv, cs, cs, 8, 4, 128)
    n = 64 * 1024 * 1024
    p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    adam_flat(p, g, m, v, torch.empty(n, device="cuda", dtype=torch.bfloat16), 1e-4, 0.9, 0.95, 1e-8, 0.1, 1)
    lg = torch.randn(2048, 1, 128256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    t = torch.randint(0, 128256, (2048, 1), device="cuda")
    loss = fused_vocab_parallel_cross_entropy(lg * 1.0, t)
    loss.sum().backward()
    torch.cuda.synchronize()


def fp8():
    from ..ops import gemm as G
    from ..ops import gemm_fp8 as F
    from ..ops.quant import quant_128x128, quant_1x128
    M = N = K = 8192
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    xq, xs = quant_1x128(x)
    wq, ws = quant_128x128(w)
    del x, w
    import time
    for _ in range(3):
        F.fp8_gemm(xq, xs, wq, ws)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        F.fp8_gemm(xq, xs, wq, ws)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    print(f"fp8 blockscaled 8192^3: {ms:.3f} ms  {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s (back-to-back launches, L2 warm)")
    G.check_status()


def gemm_tp8():
    from ..ops import gemm as G
    for (M, N, K) in ((8192, 768, 4096), (8192, 3584, 4096), (8192, 4096, 1792), (8192, 4096, 512)):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        for _ in range(2):
            G.linear_fwd(x, w)
    torch.cuda.synchronize()
    G.check_status()


def flash():
    """Two launches each of the flash-attention forward and backward kernels: seq 4096, 8 query / 2 KV heads, causal."""
    from ..ops import gemm as G
    from ..ops.flash_sm100_impl import flash_bwd, flash_fwd
    s, nq, nkv = 4096, 8, 2
    q = torch.randn(s, 1, nq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(s, 1, nkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(s, 1, nkv, 128, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(s, 1, nq, 128, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        o, lse = flash_fwd(q, k, v, True, 128 ** -0.5)
        flash_bwd(do, q, k, v, o, lse, True, 128 ** -0.5)
    torch.cuda.synchronize()
    G.check_status()


if __name__ == "__main__":
    {"gemm": gemm, "elementwise": elementwise, "fp8": fp8, "gemm_tp8": gemm_tp8, "flash": flash}[sys.argv[1] if len(sys.argv) > 1 else "gemm"]()
