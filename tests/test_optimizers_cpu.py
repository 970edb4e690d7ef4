import torch


def test_newton_schulz_orthogonalises():
    from mindspeed_b200.optimizer.muon import newton_schulz
    torch.manual_seed(0)
    for shape in ((64, 32), (32, 96)):
        x = torch.randn(*shape)
        for ct, steps, tol in (("quintic", 6, 0.35), ("polar_express", 8, 0.05)):
            o = newton_schulz(x, steps, ct)
            s = torch.linalg.svdvals(o)
            assert (s - 1).abs().max() < tol, (shape, ct, s.min(), s.max())
        # same subspace: U V^T of the SVD
        u, _, vt = torch.linalg.svd(x, full_matrices=False)
        o = newton_schulz(x, 8, "polar_express")
        assert (o - u @ vt).abs().max() < 0.05


def test_muon_descends_on_quadratic():
    from mindspeed_b200.optimizer.muon import Muon
    torch.manual_seed(1)
    w = torch.nn.Parameter(torch.randn(16, 16))
    target = torch.randn(16, 16)
    opt = Muon([w], lr=0.1, momentum=0.9, nesterov=True)
    first = None
    for _ in range(120):
        loss = (w - target).pow(2).sum()
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.2 * first


def test_adamw_matches_torch():
    from mindspeed_b200.optimizer import AdamW
    torch.manual_seed(2)
    a = torch.nn.Parameter(torch.randn(33, 7))
    b = torch.nn.Parameter(a.detach().clone())
    o1 = AdamW([a], lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1)
    o2 = torch.optim.AdamW([b], lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1)
    for _ in range(4):
        g = torch.randn(33, 7)
        a.grad, b.grad = g.clone(), g.clone()
        o1.step(); o2.step()
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_blockwise_and_mx_quant_roundtrip():
    from mindspeed_b200.ops import quant as Q
    torch.manual_seed(3)
    x = torch.randn(256, 512) * torch.logspace(-3, 2, 512)
    q, s = Q.quant_1x128(x)
    back = (q.float().view(256, 4, 128) * s.unsqueeze(-1)).view(256, 512)
    assert ((back - x).abs() <= x.abs().view(256, 4, 128).amax(-1, keepdim=True).expand(256, 4, 128).reshape(256, 512) * 0.07).all()
    w = torch.randn(256, 512)
    wq, ws = Q.quant_128x128(w)
    y = Q.fp8_blockwise_matmul_ref(q, s, wq, ws, torch.float32)
    ref = x @ w.t()
    assert (y - ref).abs().max() / ref.abs().max() < 0.05
    mq, e = Q.quant_mx(x, axis=-1)
    assert e.dtype == torch.uint8
    assert (Q.dequant_mx(mq, e) - x).abs().max() / x.abs().max() < 0.07
    q1, s1 = Q.quantize_blockwise(torch.randn(1000), 128)
    assert q1.numel() == 1024 and s1.numel() == 8
