"""tcgen05 flash attention forward (and its backward pairing) against the fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kernel", [1, 2])
@pytest.mark.parametrize("sq,b,nq,nkv,causal", [(128, 1, 1, 1, False), (256, 1, 2, 1, True), (512, 2, 4, 2, True),
                                                 (1024, 1, 8, 2, True), (384, 1, 2, 2, False), (2048, 1, 4, 1, True)])
def test_flash_fwd_matches_reference(sq, b, nq, nkv, causal, kernel):
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.ops.flash_sm100_impl import flash_fwd
    torch.manual_seed(0)
    q = torch.randn(sq, b, nq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sq, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sq, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    o, lse = flash_fwd(q, k, v, causal, scale, kernel=kernel)
    torch.cuda.synchronize()
    G.check_status()
    ro, rl = attention_ref(q, k, v, causal, scale, return_lse=True)
    torch.testing.assert_close(o.float(), ro.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse, rl, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("sq,sk,causal", [(200, 200, True), (300, 520, False), (128, 640, True), (640, 384, False), (72, 1000, True)])
def test_flash_fwd2_ragged_lengths_and_offsets(sq, sk, causal):
    """Lengths that are not multiples of the tile sizes, and more keys than queries (causal rows then see the keys up to
    their own position counted from the end, as in chunked prefill); scores with a large spread so the running maximum
    moves by more than the lazy-rescale threshold."""
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.ops.flash_sm100_impl import flash_fwd
    torch.manual_seed(3)
    b, nq, nkv = 2, 4, 2
    q = torch.randn(sq, b, nq, 128, device="cuda", dtype=torch.bfloat16) * 2.0
    k = torch.randn(sk, b, nkv, 128, device="cuda", dtype=torch.bfloat16) * 2.0
    k[sk // 2:] *= 3.0                        # later keys score much higher: forces rescales of the running output
    v = torch.randn(sk, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    if causal and sk < sq:
        pytest.skip("causal needs at least as many keys as queries")
    o, lse = flash_fwd(q, k, v, causal, scale)
    torch.cuda.synchronize()
    G.check_status()
    ro, rl = attention_ref(q, k, v, causal, scale, return_lse=True, q_offset=(sk - sq) if causal else 0)
    torch.testing.assert_close(o.float(), ro.float(), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(lse, rl, atol=2e-2, rtol=1e-3)


def test_flash_strided_packed_qkv_and_backward():
    """q/k/v as strided views of a packed QKV activation; gradients through the wrapper match the reference."""
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.ops.flash_sm100_impl import flash_attention
    torch.manual_seed(1)
    s, b, ng, qpg, d = 256, 1, 2, 2, 128
    qkv = torch.randn(s, b, ng, qpg + 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q = qkv[:, :, :, :qpg].reshape(s, b, ng * qpg, d)
    k, v = qkv[:, :, :, qpg], qkv[:, :, :, qpg + 1]
    out = flash_attention(q, k, v, True, None, False)
    w = torch.randn_like(out)
    (out.float() * w.float()).sum().backward()
    torch.cuda.synchronize()
    G.check_status()
    ref_in = qkv.detach().float().requires_grad_(True)
    rq = ref_in[:, :, :, :qpg].reshape(s, b, ng * qpg, d)
    ro = attention_ref(rq, ref_in[:, :, :, qpg], ref_in[:, :, :, qpg + 1], True)
    (ro * w.float()).sum().backward()
    torch.testing.assert_close(out.float(), ro, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(qkv.grad.float(), ref_in.grad, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("sq,sk,b,nq,nkv,causal", [(128, 128, 1, 1, 1, False), (256, 256, 1, 2, 1, True), (512, 512, 2, 4, 2, True),
                                                   (1024, 1024, 1, 8, 2, True), (384, 640, 1, 2, 2, False), (200, 200, 1, 2, 1, True),
                                                   (128, 512, 1, 4, 4, True), (2048, 2048, 1, 4, 1, True)])
def test_flash_bwd_matches_reference(sq, sk, b, nq, nkv, causal):
    """dQ, dK, dV of the tcgen05 backward against the fp32 reference backward (same O and LSE)."""
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.attention import attention_ref, attn_bwd_ref
    from mindspeed_b200.ops.flash_sm100_impl import flash_bwd, flash_fwd
    torch.manual_seed(4)
    q = torch.randn(sq, b, nq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sk, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sk, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(sq, b, nq, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    off = (sk - sq) if causal else 0
    o, lse = flash_fwd(q, k, v, causal, scale)
    dq, dk, dv = flash_bwd(do, q, k, v, o, lse, causal, scale)
    torch.cuda.synchronize()
    G.check_status()
    ro, rl = attention_ref(q, k, v, causal, scale, return_lse=True, q_offset=off)
    rdq, rdk, rdv = attn_bwd_ref(do, q, k, v, ro, rl, causal, scale, q_offset=off)
    for name, got, ref in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        ref = ref.float()
        err = (got.float() - ref).abs().max().item()
        assert err < 3e-2 * max(1.0, ref.abs().max().item()), (name, err, ref.abs().max().item())
        torch.testing.assert_close(got.float(), ref, atol=4e-2 * ref.abs().max().item(), rtol=5e-2)
