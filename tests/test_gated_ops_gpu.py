"""CUDA gated RMSNorm and Sinkhorn kernels against their fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,rows,cols", [(torch.float32, 37, 96), (torch.bfloat16, 4096, 2048), (torch.bfloat16, 130, 128)])
def test_gated_norm_forward_backward(dtype, rows, cols):
    from mindspeed_b200.ops import gated_ops as GO
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", dtype=dtype, requires_grad=True)
    g = torch.randn(rows, cols, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype).requires_grad_(True)
    dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
    y = GO.rms_norm_gated(x, g, w)
    gx, gg, gw = torch.autograd.grad(y, (x, g, w), dy)
    xr, gr, wr = (t.detach().float().requires_grad_(True) for t in (x, g, w))
    yr = GO.rms_norm_gated_ref(xr, gr, wr)
    rx, rg, rw = torch.autograd.grad(yr, (xr, gr, wr), dy.float())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    rel = lambda a, b: ((a.float() - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()
    assert rel(y, yr) < tol and rel(gx, rx) < tol and rel(gg, rg) < tol and rel(gw, rw) < max(tol, 1e-4)


@pytest.mark.parametrize("n,iters", [(4, 20), (8, 5), (2, 32)])
def test_sinkhorn_forward_backward(n, iters):
    from mindspeed_b200.ops import gated_ops as GO
    torch.manual_seed(1)
    lg = torch.randn(300, 5, n, n, device="cuda", requires_grad=True)
    out = GO.sinkhorn(lg, iters)
    ref_in = lg.detach().clone().requires_grad_(True)
    ref = GO.sinkhorn_ref(ref_in, iters)
    assert torch.allclose(out, ref, atol=1e-5)
    dout = torch.randn_like(out)
    (g1,) = torch.autograd.grad(out, lg, dout)
    (g2,) = torch.autograd.grad(ref, ref_in, dout)
    assert torch.allclose(g1, g2, atol=2e-4), (g1 - g2).abs().max()
