"""tcgen05 GEMM against an fp32 reference: all operand layouts, edge tiles, epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())


SHAPES = [(128, 256, 64), (256, 512, 128), (1000, 776, 520), (8192, 768, 512), (384, 128, 4096), (130, 264, 72)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_fwd(M, N, K):
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    y = G.linear_fwd(x, w)
    torch.cuda.synchronize()
    G.check_status()
    ref = x.float() @ w.float().t()
    assert _rel(y, ref) < 1e-2, _rel(y, ref)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_dgrad(M, N, K):
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(1)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    dx = G.linear_dgrad(dy, w)
    torch.cuda.synchronize()
    G.check_status()
    ref = dy.float() @ w.float()
    assert _rel(dx, ref) < 1e-2, _rel(dx, ref)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_wgrad(M, N, K):
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(2)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    ref = dy.float().t() @ x.float()
    dw = G.linear_wgrad(dy, x)
    acc = torch.ones(N, K, device="cuda", dtype=torch.float32)
    G.linear_wgrad(dy, x, acc)
    G.linear_wgrad(dy, x, acc)
    torch.cuda.synchronize()
    G.check_status()
    assert _rel(dw, ref) < 1e-2
    assert _rel(acc, 1 + 2 * ref) < 1e-2


def test_bias_epilogue_and_determinism():
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(3)
    x = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(768, device="cuda", dtype=torch.bfloat16)
    y1 = G.linear_fwd(x, w, bias=b)
    y2 = G.linear_fwd(x, w, bias=b)
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(y1, y2)
    assert _rel(y1, x.float() @ w.float().t() + b.float()) < 1e-2
