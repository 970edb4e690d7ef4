"""tcgen05 GEMM against an fp32 reference: all operand layouts, edge tiles, epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())


def _elementwise(y, ref, k):
    """Every element against the fp32 result rounded to the output type: two units in the last place of bf16, plus an
    absolute term for elements that cancel to near zero (fp32 accumulation order over ``k`` products)."""
    want = ref.to(y.dtype).float() if y.dtype != torch.float32 else ref
    rtol = 2.0 ** -7 if y.dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(y.float(), want, rtol=rtol, atol=1e-5 * k + 1e-3)


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
    _elementwise(y, ref, K)


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
    _elementwise(dx, ref, N)


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
    _elementwise(dw, ref, M)
    _elementwise(acc, 1 + 2 * ref, 2 * M)


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


EDGE = [(130, 264, 72), (1000, 776, 520), (300, 136, 200), (256, 256, 64), (8192, 768, 512)]


@pytest.mark.parametrize("v", [1, 2, 3])
@pytest.mark.parametrize("M,N,K", EDGE)
def test_every_kernel_variant_elementwise(v, M, N, K):
    """Each kernel (one-CTA, CTA pair 256x256, CTA pair 256x128) against the fp32 product rounded to bf16, element by
    element, on shapes with ragged M / N / K tiles; weight-gradient accumulation into fp32 twice."""
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(10 + v)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.full((N, K), 0.5, device="cuda", dtype=torch.float32)
    f32 = torch.empty(M, N, device="cuda", dtype=torch.float32)
    with G.variant(v):
        y = G.linear_fwd(x, w)
        dx = G.linear_dgrad(dy, w)
        dw = G.linear_wgrad(dy, x)
        G.linear_wgrad(dy, x, acc)
        G.linear_wgrad(dy, x, acc)
        G._gemm(x, w, f32, M, N, K, K, K, N, 0, 0, G.EPI_F32)
    torch.cuda.synchronize()
    G.check_status()
    # fp32 accumulation order differs from the reference's: allow one bf16 ulp of the result (2^-8 relative) plus a
    # small absolute term for cancellation
    for got, ref in ((y, x.float() @ w.float().t()), (dx, dy.float() @ w.float()), (dw, dy.float().t() @ x.float())):
        torch.testing.assert_close(got.float(), ref, rtol=8e-3, atol=2e-2 * ref.abs().mean().item())
    torch.testing.assert_close(f32, x.float() @ w.float().t(), rtol=1e-4, atol=1e-3 * (K ** 0.5))
    torch.testing.assert_close(acc, 0.5 + 2 * (dy.float().t() @ x.float()), rtol=1e-4, atol=2e-3 * (M ** 0.5))


def test_pair_kernel_bias_and_strided_output():
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(5)
    x = torch.randn(640, 320, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(200, 320, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(200, device="cuda", dtype=torch.bfloat16)
    with G.variant(2):
        y = G.linear_fwd(x, w, bias=b)
    torch.cuda.synchronize()
    G.check_status()
    torch.testing.assert_close(y.float(), x.float() @ w.float().t() + b.float(), rtol=8e-3, atol=0.3)


def test_weight_gradient_accumulation_reproducible_without_stream_k():
    from mindspeed_b200.ops import gemm as G
    torch.manual_seed(6)
    dy = torch.randn(4096, 1536, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    ref = dy.float().t() @ x.float()
    outs = []
    G.set_stream_k(False)
    try:
        for _ in range(2):
            acc = torch.zeros(1536, 1024, device="cuda", dtype=torch.float32)
            G.linear_wgrad(dy, x, acc)
            outs.append(acc)
    finally:
        G.set_stream_k(True)
    acc = torch.zeros(1536, 1024, device="cuda", dtype=torch.float32)
    G.linear_wgrad(dy, x, acc)                      # k-block balanced: same value up to fp32 summation order
    torch.cuda.synchronize()
    G.check_status()
    assert torch.equal(outs[0], outs[1])
    torch.testing.assert_close(outs[0], ref, rtol=1e-4, atol=0.05)
    torch.testing.assert_close(acc, ref, rtol=1e-4, atol=0.05)


@pytest.mark.parametrize("sizes,K,N", [([300, 0, 37, 512, 64, 129], 256, 384), ([1000, 2000, 17, 983], 512, 1024), ([5, 3], 64, 128),
                                       ([256] * 8, 1024, 512)])
def test_grouped_gemm_forward_and_gradients(sizes, K, N):
    """One launch per direction over all experts, row ranges taken from a device tensor; ragged expert boundaries, empty
    and tiny experts; weight gradient both as a returned tensor and accumulated into an fp32 main_grad."""
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.grouped_gemm import grouped_gemm
    torch.manual_seed(7)
    E, R = len(sizes), sum(sizes)
    x = (torch.randn(R + 40, K, device="cuda") * 0.5).bfloat16().requires_grad_(True)     # 40 spare rows past the last expert
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    counts = torch.tensor(sizes, device="cuda", dtype=torch.int64)
    y = grouped_gemm(x, w, counts)
    dy = torch.randn(R + 40, N, device="cuda").bfloat16()
    dy[R:] = 0
    (y[:R].float() * dy[:R].float()).sum().backward()
    torch.cuda.synchronize()
    G.check_status()
    xf, wf = x.detach().float(), w.detach().float()
    ry = torch.zeros(R, N, device="cuda")
    rdx = torch.zeros(R, K, device="cuda")
    rdw = torch.zeros(E, K, N, device="cuda")
    s = 0
    for e, n in enumerate(sizes):
        ry[s:s + n] = xf[s:s + n] @ wf[e]
        rdx[s:s + n] = dy[s:s + n].float() @ wf[e].t()
        rdw[e] = xf[s:s + n].t() @ dy[s:s + n].float()
        s += n
    torch.testing.assert_close(y[:R].float(), ry, rtol=1e-2, atol=2e-2 * ry.abs().mean().item() + 1e-3)
    torch.testing.assert_close(x.grad[:R].float(), rdx, rtol=1e-2, atol=2e-2 * rdx.abs().mean().item() + 1e-3)
    torch.testing.assert_close(w.grad.float(), rdw, rtol=1e-2, atol=2e-2 * rdw.abs().mean().item() + 1e-3)
    # accumulate into main_grad twice
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.full((E, K, N), 0.25, device="cuda", dtype=torch.float32)
    for _ in range(2):
        y2 = grouped_gemm(x.detach(), w2, counts)
        (y2[:R].float() * dy[:R].float()).sum().backward()
    torch.cuda.synchronize()
    G.check_status()
    torch.testing.assert_close(w2.main_grad, 0.25 + 2 * rdw, rtol=1e-3, atol=2e-3 * rdw.abs().mean().item() + 1e-3)
