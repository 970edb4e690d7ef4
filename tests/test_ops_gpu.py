"""sm_100a elementwise / reduction kernels against fp32 PyTorch references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.float16: 1e-3, torch.bfloat16: 5e-3}


def _close(a, b, dtype, scale=1.0):
    tol = TOL[dtype] * scale
    torch.testing.assert_close(a.float(), b.float(), atol=tol * max(1.0, b.float().abs().max().item()), rtol=tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 512), (7, 520), (4, 12288), (1000, 1024), (2500, 4096), (700, 8192),
                                       (300, 16384), (5, 20000), (9, 1028)])
def test_rmsnorm(dtype, rows, cols):
    from mindspeed_b200.ops.norm import rms_norm, rms_norm_ref
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype).requires_grad_(True)
    y = rms_norm(x, w, 1e-5)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = rms_norm_ref(xr, wr, 1e-5)
    _close(y, yr, dtype)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    _close(x.grad, xr.grad, dtype, 2)
    _close(w.grad, wr.grad, dtype, 4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols,zc", [(2500, 4096, False), (333, 1024, True), (64, 8192, False), (5, 20000, False)])
def test_add_rmsnorm(dtype, rows, cols, zc):
    """Residual add fused with the norm: both outputs and all three gradients, with a gradient on each output."""
    from mindspeed_b200.ops.norm import add_rms_norm, rms_norm_ref
    torch.manual_seed(3)
    x = torch.randn(rows, cols, device="cuda", dtype=dtype, requires_grad=True)
    r = torch.randn(rows, cols, device="cuda", dtype=dtype, requires_grad=True)
    w = (0.1 * torch.randn(cols, device="cuda") + (0.0 if zc else 1.0)).to(dtype).requires_grad_(True)
    h, y = add_rms_norm(x, r, w, 1e-5, zc)
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    # the kernel normalises the sum rounded to the tensor type (straight-through for the gradient)
    hr = (xr + rr) + ((xr + rr).to(dtype).float() - (xr + rr)).detach()
    yr = rms_norm_ref(hr, wr, 1e-5, zc)
    _close(h, hr, dtype)
    _close(y, yr, dtype)
    gh, gy = torch.randn_like(h), torch.randn_like(y)
    torch.autograd.backward([h, y], [gh, gy])
    torch.autograd.backward([hr, yr], [gh.float(), gy.float()])
    _close(x.grad, xr.grad, dtype, 2)
    _close(r.grad, rr.grad, dtype, 2)
    _close(w.grad, wr.grad, dtype, 6)
    # only the norm output is used downstream
    x.grad = r.grad = w.grad = None
    h2, y2 = add_rms_norm(x, r, w, 1e-5, zc)
    y2.backward(gy)
    xr.grad = None
    rms_norm_ref((xr + rr) + ((xr + rr).to(dtype).float() - (xr + rr)).detach(), wr, 1e-5, zc).backward(gy.float())
    _close(x.grad, xr.grad, dtype, 2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    from mindspeed_b200.ops.activation import swiglu, swiglu_ref
    torch.manual_seed(1)
    x = torch.randn(129, 2 * 1792, device="cuda", dtype=dtype, requires_grad=True)
    y = swiglu(x)
    xr = x.detach().float().requires_grad_(True)
    yr = swiglu_ref(xr)
    _close(y, yr, dtype)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    _close(x.grad, xr.grad, dtype, 2)


def test_swiglu_weighted():
    from mindspeed_b200.ops.activation import swiglu, swiglu_ref
    torch.manual_seed(2)
    x = torch.randn(77, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    sc = torch.rand(77, device="cuda", requires_grad=True)
    y = swiglu(x, sc)
    xr, sr = x.detach().float().requires_grad_(True), sc.detach().clone().requires_grad_(True)
    yr = swiglu_ref(xr, sr)
    _close(y, yr, torch.bfloat16)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    _close(x.grad, xr.grad, torch.bfloat16, 2)
    _close(sc.grad, sr.grad, torch.bfloat16, 4)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("s,b,d", [(96, 2, 128), (97, 1, 128), (33, 3, 64), (20, 1, 96), (1031, 1, 256)])
def test_rope(interleaved, s, b, d):
    from mindspeed_b200.ops.rope import apply_rope, apply_rope_ref, rope_packed_qkv_
    torch.manual_seed(3)
    n = 6
    ang = torch.outer(torch.arange(s, device="cuda").float(), 1.0 / (10000 ** (torch.arange(0, d, 2, device="cuda").float() / d)))
    emb = torch.stack((ang, ang), -1).reshape(s, d) if interleaved else torch.cat((ang, ang), -1)
    cos, sin = emb.cos().contiguous(), emb.sin().contiguous()
    t = torch.randn(s, b, n, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = apply_rope(t, cos, sin, interleaved)
    tr = t.detach().float().requires_grad_(True)
    yr = apply_rope_ref(tr, cos, sin, interleaved)
    _close(y, yr, torch.bfloat16)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    _close(t.grad, tr.grad, torch.bfloat16)
    # packed qkv in place: groups=2, 3 q heads per group
    groups, qpg = 2, 3
    qkv = torch.randn(s, b, groups * (qpg + 2) * d, device="cuda", dtype=torch.bfloat16)
    ref = qkv.clone().view(s, b, groups, qpg + 2, d)
    part = ref[:, :, :, :qpg + 1].reshape(s, b, groups * (qpg + 1), d)
    ref[:, :, :, :qpg + 1] = apply_rope_ref(part.float(), cos, sin, interleaved).to(torch.bfloat16).view(s, b, groups, qpg + 1, d)
    rope_packed_qkv_(qkv, cos, sin, groups, qpg, d, interleaved)
    _close(qkv.view_as(ref), ref, torch.bfloat16)


def test_adam_flat_matches_torch_adamw():
    from mindspeed_b200.ops.adam import adam_flat
    torch.manual_seed(4)
    n = 100003
    p = torch.randn(n, device="cuda")
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = g.clone()
        opt.step()
        adam_flat(p, g, m, v, p16, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(p, ref.data, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(p16.float(), p.bfloat16().float())


def test_l2norm_and_clip():
    from mindspeed_b200.ops import adam as A
    g = torch.randn(1 << 20, device="cuda")
    out = A.l2norm_sq(g)
    torch.testing.assert_close(out.item(), g.double().pow(2).sum().item(), rtol=1e-4, atol=0)
    coef = torch.zeros(1, device="cuda"); inf = torch.zeros(1, device="cuda"); nrm = torch.zeros(1, device="cuda")
    A.clip_coef(out, 1.0, coef, inf, nrm)
    assert abs(coef.item() - 1.0 / (g.norm().item() + 1e-6)) < 1e-6 and inf.item() == 0


@pytest.mark.parametrize("vocab", [4096, 16032, 1000])
def test_fused_cross_entropy(vocab):
    from mindspeed_b200.ops.cross_entropy import fused_vocab_parallel_cross_entropy
    torch.manual_seed(5)
    rows = 257
    logits = (3 * torch.randn(rows, 1, vocab, device="cuda")).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, vocab, (rows, 1), device="cuda")
    ref_in = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in.view(rows, vocab), tgt.view(-1), reduction="none")
    x = logits.detach().clone().requires_grad_(True)
    y = x * 1.0
    loss = fused_vocab_parallel_cross_entropy(y, tgt)
    torch.testing.assert_close(loss.view(-1), ref, atol=2e-2, rtol=1e-2)
    w = torch.rand(rows, 1, device="cuda")
    (loss * w).sum().backward()
    (ref * w.view(-1)).sum().backward()
    torch.testing.assert_close(x.grad.float(), ref_in.grad, atol=5e-3, rtol=5e-2)


def test_reuse_fp32_param_split_merge_and_adam():
    from mindspeed_b200.memory.reuse_param import adam_flat_reuse, merge_fp32, split_fp32
    from mindspeed_b200.ops.adam import adam_flat
    torch.manual_seed(6)
    n = 70001
    p = torch.randn(n, device="cuda")
    hi, lo = split_fp32(p)
    assert torch.equal(merge_fp32(hi, lo), p)                       # exact round trip
    assert (hi.float() - p).abs().max() <= p.abs().max() * 2 ** -8  # hi is the rounded bf16 of the master
    ref = p.clone()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    m2, v2 = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        adam_flat(ref, g, m, v, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
        adam_flat_reuse(hi, lo, g, m2, v2, 1e-3, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(merge_fp32(hi, lo), ref, atol=1e-6, rtol=1e-5)


def test_scaled_masked_softmax_and_ring_update_and_quant():
    from mindspeed_b200.ops import misc
    from mindspeed_b200.ops import quant as Q
    torch.manual_seed(7)
    x = torch.randn(2, 3, 64, 96, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    mask = torch.rand(2, 1, 64, 96, device="cuda") > 0.7
    mask[..., 0] = False
    y = misc.scaled_masked_softmax(x, mask, 0.5)
    xr = x.detach().float().requires_grad_(True)
    yr = misc.scaled_masked_softmax_ref(xr, mask, 0.5)
    torch.testing.assert_close(y.float(), yr.float(), atol=1e-2, rtol=1e-2)
    g = torch.randn_like(y)
    y.backward(g); yr.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=2e-2, rtol=5e-2)
    yc = misc.scaled_masked_softmax(x.detach(), None, 1.0, causal=True)
    torch.testing.assert_close(yc.float(), misc.scaled_masked_softmax_ref(x.detach(), None, 1.0, True).float(), atol=1e-2, rtol=1e-2)
    rows, d = 1000, 128
    po, co = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16), torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
    pm, cm = torch.randn(rows, device="cuda"), torch.randn(rows, device="cuda")
    ps_, cs = torch.rand(rows, device="cuda") + 0.1, torch.rand(rows, device="cuda") + 0.1
    o, m, l = misc.ring_attention_update(po, pm, ps_, co, cm, cs)
    ro, rm, rl = misc.ring_attention_update_ref(po, pm, ps_, co, cm, cs)
    torch.testing.assert_close(o.float(), ro.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(m, rm); torch.testing.assert_close(l, rl, rtol=1e-4, atol=1e-5)
    w = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16) * 3
    q, s = misc.quant_1x128(w)
    qr, sr = Q.quant_1x128(w)
    torch.testing.assert_close(s, sr, rtol=1e-5, atol=0)
    assert (q.float() - qr.float()).abs().max() <= 32          # at most one fp8 step apart (rounding of the division)
    h, yn = misc.add_rmsnorm(po, co, torch.ones(d, device="cuda", dtype=torch.bfloat16))
    torch.testing.assert_close(h, po + co)


@pytest.mark.parametrize("experts", [False, True])
def test_fused_ffn_op(experts):
    """ffn(): both GEMMs on the tcgen05 kernels (dense or one grouped launch), SwiGLU on the fused kernel."""
    from mindspeed_b200.ops.ffn import ffn
    torch.manual_seed(5)
    K, Fh, N = 512, 768, 256
    if experts:
        counts = [300, 0, 129, 451]
        x = torch.randn(sum(counts), K, device="cuda", dtype=torch.bfloat16)
        w1 = (torch.randn(4, K, 2 * Fh, device="cuda") * 0.05).bfloat16()
        w2 = (torch.randn(4, Fh, N, device="cuda") * 0.05).bfloat16()
        y = ffn(x, w1, w2, "swiglu", expert_tokens=torch.tensor(counts, device="cuda"))
        outs, r = [], 0
        for e, n in enumerate(counts):
            h = x[r:r + n].float() @ w1[e].float()
            outs.append((torch.nn.functional.silu(h[:, :Fh]) * h[:, Fh:]).bfloat16().float() @ w2[e].float())
            r += n
        ref = torch.cat(outs)
    else:
        x = torch.randn(640, K, device="cuda", dtype=torch.bfloat16)
        w1 = (torch.randn(K, 2 * Fh, device="cuda") * 0.05).bfloat16()
        w2 = (torch.randn(Fh, N, device="cuda") * 0.05).bfloat16()
        y = ffn(x, w1, w2, "swiglu")
        h = x.float() @ w1.float()
        ref = (torch.nn.functional.silu(h[:, :Fh]) * h[:, Fh:]).bfloat16().float() @ w2.float()
    torch.cuda.synchronize()
    _close(y, ref, torch.bfloat16, 4)
