"""Small, self-terminating workloads for Nsight Compute captures of single kernels.

  python -m mindspeed_b200.ops.ncu_targets gemm        # 3 launches each of fwd / dgrad / wgrad, 8192^3 bf16
  python -m mindspeed_b200.ops.ncu_targets elementwise # rmsnorm / swiglu / rope / adam / cross-entropy once each

Inputs exceed the 126 MB L2 but stay well under 2 GB on the device; there are only a handful of launches, so a
``--set full`` capture ends by itself within a minute or two.
"""
import sys

import torch


def gemm():
    from . import gemm as G
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
    from .activation import swiglu
    from .adam import adam_flat
    from .cross_entropy import fused_vocab_parallel_cross_entropy
    from .norm import rms_norm
    from .rope import rope_packed_qkv_
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


if __name__ == "__main__":
    {"gemm": gemm, "elementwise": elementwise}[sys.argv[1] if len(sys.argv) > 1 else "gemm"]()
