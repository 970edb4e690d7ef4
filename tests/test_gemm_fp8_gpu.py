"""Block-scaled fp8 tcgen05 GEMM against the fp32 evaluation of the same quantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _quant(M, N, K, a_dtype=torch.float8_e4m3fn):
    from mindspeed_b200.ops.quant import quant_128x128, quant_1x128
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 3
    w = torch.randn(N, K, device="cuda") * 0.05
    xq, xs = quant_1x128(x, dtype=a_dtype)
    wq, ws = quant_128x128(w)
    return x, w, xq, xs, wq, ws


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 256, 1024), (4096, 1536, 4096), (77, 128, 256)])
def test_plain_matches_reference(M, N, K):
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops import gemm_fp8 as F
    x, w, xq, xs, wq, ws = _quant(M, N, K)
    y = F.fp8_gemm(xq, xs, wq, ws)
    torch.cuda.synchronize()
    G.check_status()
    ref = F._ref(xq, xs, wq, ws, False, torch.float32)
    err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-2, err                         # bf16 output rounding only: the operands are identical
    full = (x @ w.t())
    assert ((y.float() - full).norm() / full.norm()).item() < 0.08      # and the recipe itself is a sane approximation


def test_e5m2_gradients_rowwise_scales_and_fp32_accumulate():
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops import gemm_fp8 as F
    from mindspeed_b200.ops.quant import quant_1x128
    torch.manual_seed(1)
    a = torch.randn(384, 512, device="cuda")
    b = torch.randn(200, 512, device="cuda")            # N = 200: not a multiple of 128, row-wise scales allow it
    aq, as_ = quant_1x128(a, dtype=torch.float8_e5m2)
    bq, bs = quant_1x128(b)
    acc = torch.ones(384, 200, device="cuda", dtype=torch.float32)
    F.fp8_gemm(aq, as_, bq, bs, w_rowwise=True, out=acc, accumulate=True)
    torch.cuda.synchronize()
    G.check_status()
    ref = 1.0 + F._ref(aq, as_, bq, bs, True, torch.float32)
    assert (acc - ref).abs().max().item() < 1e-3 * ref.abs().max().item()


def test_grouped_matches_per_expert_reference():
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops import gemm_fp8 as F
    from mindspeed_b200.ops.quant import quant_128x128, quant_1x128
    torch.manual_seed(2)
    counts = [300, 0, 129, 5]
    K, N = 512, 256
    x = torch.randn(sum(counts), K, device="cuda")
    w = torch.randn(len(counts), N, K, device="cuda") * 0.05
    xq, xs = quant_1x128(x)
    qs = [quant_128x128(w[g]) for g in range(len(counts))]
    wq, ws = torch.stack([q[0] for q in qs]), torch.stack([q[1] for q in qs])
    y = F.fp8_grouped_gemm(xq, xs, wq, ws, counts)
    torch.cuda.synchronize()
    G.check_status()
    s = 0
    for g, c in enumerate(counts):
        ref = F._ref(xq[s:s + c], xs[s:s + c], wq[g], ws[g], False, torch.float32)
        if c:
            assert (y[s:s + c].float() - ref).abs().max().item() < 1e-2 * ref.abs().max().item(), g
        s += c


def test_fp8_linear_autograd_on_gpu():
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.gemm_fp8 import fp8_blockwise_linear
    torch.manual_seed(3)
    x = (torch.randn(4, 100, 256, device="cuda")).bfloat16().requires_grad_(True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    cache = {}
    y = fp8_blockwise_linear(x, w, cache)
    g = torch.randn_like(y)
    y.backward(g)
    torch.cuda.synchronize()
    G.check_status()
    ref = x.float() @ w.float().t()
    gx = g.float() @ w.float()
    gw = g.float().reshape(-1, 384).t() @ x.float().reshape(-1, 256)
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y, ref) < 0.08 and rel(x.grad, gx) < 0.08 and rel(w.grad, gw) < 0.08
    assert set(cache) == {"wq", "ws", "wtq", "wts"}
