"""Fused FFN op and quantised grouped GEMMs against their definitions."""
import pytest
import torch
import torch.nn.functional as F


@pytest.mark.parametrize("activation", ["gelu", "swiglu", "geglu", "relu"])
def test_ffn_dense_and_experts(activation):
    from mindspeed_b200.ops.ffn import ffn
    torch.manual_seed(0)
    gated = activation in ("swiglu", "geglu")
    act = {"gelu": F.gelu, "relu": F.relu, "swiglu": F.silu, "geglu": F.gelu}[activation]
    x = torch.randn(3, 5, 16)
    w1, w2 = torch.randn(16, 24 * (2 if gated else 1)) * 0.2, torch.randn(24, 8) * 0.2
    b1, b2 = torch.randn(w1.shape[1]) * 0.1, torch.randn(8) * 0.1
    h = x @ w1 + b1
    ref = ((act(h[..., :24]) * h[..., 24:]) if gated else act(h)) @ w2 + b2
    torch.testing.assert_close(ffn(x, w1, w2, activation, bias1=b1, bias2=b2), ref, rtol=1e-5, atol=1e-5)
    # experts: rows sorted by expert, per-expert weights and biases
    counts = [4, 0, 7, 4]
    xe = torch.randn(sum(counts), 16)
    W1, W2 = torch.randn(4, 16, w1.shape[1]) * 0.2, torch.randn(4, 24, 8) * 0.2
    B1, B2 = torch.randn(4, w1.shape[1]) * 0.1, torch.randn(4, 8) * 0.1
    outs, r = [], 0
    for e, n in enumerate(counts):
        he = xe[r:r + n] @ W1[e] + B1[e]
        outs.append(((act(he[..., :24]) * he[..., 24:]) if gated else act(he)) @ W2[e] + B2[e])
        r += n
    got = ffn(xe, W1, W2, activation, expert_tokens=torch.tensor(counts), bias1=B1, bias2=B2)
    torch.testing.assert_close(got, torch.cat(outs), rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        ffn(x, w1, w2, "tanh")


def test_quantised_grouped_gemms():
    from mindspeed_b200.ops.ffn import quant_grouped_gemm, weight_quant_grouped_gemm
    torch.manual_seed(1)
    counts = [5, 3, 0, 8]
    x = torch.randn(16, 32)
    q = torch.randint(-127, 128, (4, 32, 12), dtype=torch.int8)
    scale, off = torch.rand(4, 12) * 0.01 + 0.001, torch.randn(4, 12).round()
    outs, r = [], 0
    for e, n in enumerate(counts):
        outs.append(x[r:r + n] @ ((q[e].float() + off[e]) * scale[e]))
        r += n
    torch.testing.assert_close(weight_quant_grouped_gemm(x, q, scale, off, counts), torch.cat(outs), rtol=1e-4, atol=1e-4)
    qx = torch.randint(-127, 128, (16, 32), dtype=torch.int8)
    tok = torch.rand(16) * 0.02
    outs, r = [], 0
    for e, n in enumerate(counts):
        outs.append((qx[r:r + n].float() @ q[e].float()) * scale[e])
        r += n
    ref = torch.cat(outs) * tok.unsqueeze(1)
    got = quant_grouped_gemm(qx, q, scale, tok, torch.tensor(counts), out_dtype=torch.float32)
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-5)


def test_dropout_add_norm_ops():
    import torch
    from mindspeed_b200.ops.norm import dropout_add_layer_norm, dropout_add_rms_norm
    g = torch.Generator().manual_seed(0)
    B, S, H = 2, 5, 16
    x0, res = torch.randn(B, S, H, generator=g), torch.randn(B, S, H, generator=g)
    w, b = torch.randn(H, generator=g), torch.randn(H, generator=g)
    rows, chans = torch.rand(B, S, generator=g), torch.rand(H, generator=g)
    # the oracle of the reference's test: scales, residual add, then the norm
    h = x0 * rows.view(B, S, 1) * chans.view(1, 1, H) + res
    rms = h / torch.sqrt((h * h).sum(-1, keepdim=True) / H + 1e-5) * w
    out, pre = dropout_add_rms_norm(x0, res, w, None, 0.0, 1e-5, rowscale=rows, layerscale=chans, prenorm=True)
    assert torch.allclose(out, rms, atol=1e-5) and torch.allclose(pre, h, atol=1e-6)
    ln = torch.nn.functional.layer_norm(x0 + res, (H,), w, b, 1e-5)
    assert torch.allclose(dropout_add_layer_norm(x0, res, w, b, 0.0, 1e-5), ln, atol=1e-5)
    assert torch.allclose(dropout_add_layer_norm(x0, None, w, b, 0.0, 1e-5), torch.nn.functional.layer_norm(x0, (H,), w, b, 1e-5), atol=1e-5)
    # dropout: the returned mask reproduces the output; kept entries are scaled by 1 / (1 - p)
    torch.manual_seed(3)
    out, pre, mask = dropout_add_rms_norm(x0, res, w, None, 0.5, 1e-5, prenorm=True, return_dropout_mask=True, residual_in_fp32=True)
    assert mask.dtype == torch.bool and 0.2 < float(mask.float().mean()) < 0.8 and pre.dtype == torch.float32
    assert torch.allclose(pre, x0 * mask / 0.5 + res, atol=1e-6)
    # evaluation mode: no dropout
    assert torch.allclose(dropout_add_layer_norm(x0, res, w, b, 0.5, 1e-5, training=False), ln, atol=1e-5)
    # differentiable
    xg = x0.clone().requires_grad_(True)
    dropout_add_rms_norm(xg, res, w, None, 0.0, 1e-5).sum().backward()
    assert torch.isfinite(xg.grad).all() and xg.grad.abs().sum() > 0
