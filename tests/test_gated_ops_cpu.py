"""Gated delta rule (chunked == recurrent), lightning indexer, Sinkhorn / hyper-connections, gated norm oracles."""
import torch

from mindspeed_b200.ops import gated_delta_rule as GD
from mindspeed_b200.ops import gated_ops as GO
from mindspeed_b200.ops import lightning_indexer as LI


def test_chunked_delta_rule_equals_recurrent_with_grads():
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 37, 3, 8, 6
    q, k = torch.randn(B, T, H, dk, dtype=torch.double), torch.randn(B, T, H, dk, dtype=torch.double)
    v = torch.randn(B, T, H, dv, dtype=torch.double)
    g = -torch.rand(B, T, H, dtype=torch.double) * 0.5
    beta = torch.rand(B, T, H, dtype=torch.double)
    S0 = torch.randn(B, H, dk, dv, dtype=torch.double) * 0.1
    for t in (q, k, v, g, beta):
        t.requires_grad_(True)
    o1, s1 = GD.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=S0, use_qk_l2norm=True)
    gr1 = torch.autograd.grad((o1 * torch.linspace(0, 1, dv, dtype=torch.double)).sum() + s1.sum(), (q, k, v, g, beta))
    for C in (8, 16, 64):
        o2, s2 = GD.gated_delta_rule_chunked(q, k, v, g, beta, initial_state=S0, chunk_size=C, use_qk_l2norm=True)
        assert torch.allclose(o1.float(), o2.float(), atol=1e-4), (C, (o1 - o2).abs().max())
        assert torch.allclose(s1.float(), s2.float(), atol=1e-4)
        gr2 = torch.autograd.grad((o2 * torch.linspace(0, 1, dv, dtype=torch.double)).sum() + s2.sum(), (q, k, v, g, beta))
        for a, b in zip(gr1, gr2):
            assert torch.allclose(a.float(), b.float(), atol=1e-3), C
    o3, s3 = GD.chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=False)
    assert s3 is None and o3.shape == (B, T, H, dv)


def test_indexer_scores_topk_and_mask():
    torch.manual_seed(1)
    B, T, H, d = 2, 50, 4, 16
    q, k, w = torch.randn(B, T, H, d), torch.randn(B, T, d), torch.rand(B, T, H)
    full = (torch.relu(torch.einsum("bthd,bsd->bths", q, k)) * w.unsqueeze(-1)).sum(2)
    sc = LI.indexer_scores(q, k, w, causal=True, block=16)
    tri = torch.tril(torch.ones(T, T, dtype=torch.bool))
    assert torch.allclose(sc[:, tri], full[:, tri], atol=1e-4) and torch.isinf(sc[:, ~tri]).all()
    idx, _ = LI.indexer_topk(q, k, w, topk=8, block=16)
    assert idx.shape == (B, T, 8)
    assert (idx[:, 0, 1:] == -1).all() and idx[:, 0, 0].eq(0).all()         # the first token sees only itself
    assert ((idx <= torch.arange(T).view(1, T, 1)) | (idx < 0)).all()
    mask = LI.sparse_attention_mask(idx, T)
    assert (torch.isfinite(mask).sum(-1)[:, 20:] == 8).all()
    probs = torch.softmax(torch.randn(B, T, T).masked_fill(~tri, float("-inf")), -1)
    loss = LI.indexer_kl_loss(sc, probs)
    assert torch.isfinite(loss) and loss > 0


def test_sinkhorn_reference_is_doubly_stochastic_and_hyper_connection_runs():
    torch.manual_seed(2)
    lg = torch.randn(5, 7, 4, 4)
    m = GO.sinkhorn(lg, iters=30)
    assert torch.allclose(m.sum(-1), torch.ones(5, 7, 4), atol=1e-3) and torch.allclose(m.sum(-2), torch.ones(5, 7, 4), atol=1e-3)
    hc = GO.HyperConnection(16, n_streams=4)
    x = torch.randn(3, 2, 16)
    streams = GO.HyperConnection.expand(x, 4)
    out = hc(streams, lambda t: torch.tanh(t))
    assert out.shape == (3, 2, 4, 16)
    # at initialisation: read = mean of identical streams = x, mixing ~ identity, write = 1  ->  every stream ~ x + f(x)
    assert torch.allclose(out[..., 0, :], x + torch.tanh(x), atol=0.05)
    out.sum().backward()
    assert hc.mix.weight.grad is not None


def test_gated_norm_backward_formulas_match_autograd():
    """The closed-form gradients the CUDA backward kernel implements, checked against autograd of the reference."""
    torch.manual_seed(3)
    x = torch.randn(6, 32, requires_grad=True)
    g = torch.randn(6, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    dy = torch.randn(6, 32)
    y = GO.rms_norm_gated_ref(x, g, w, eps=1e-6)
    gx, gg, gw = torch.autograd.grad(y, (x, g, w), dy)
    with torch.no_grad():
        r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
        xh = x * r
        sg = torch.nn.functional.silu(g)
        sig = torch.sigmoid(g)
        t = dy * sg * w
        dx = r * (t - xh * (t * xh).mean(-1, keepdim=True))
        dg = dy * xh * w * (sig * (1 + g * (1 - sig)))
        dw = (dy * sg * xh).sum(0)
    assert torch.allclose(dx, gx, atol=1e-5) and torch.allclose(dg, gg, atol=1e-5) and torch.allclose(dw, gw, atol=1e-4)
