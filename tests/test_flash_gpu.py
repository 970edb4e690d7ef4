"""tcgen05 flash attention forward (and its backward pairing) against the fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("sq,b,nq,nkv,causal", [(128, 1, 1, 1, False), (256, 1, 2, 1, True), (512, 2, 4, 2, True),
                                                 (1024, 1, 8, 2, True), (384, 1, 2, 2, False)])
def test_flash_fwd_matches_reference(sq, b, nq, nkv, causal):
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.ops.flash_sm100_impl import flash_fwd
    torch.manual_seed(0)
    q = torch.randn(sq, b, nq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sq, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sq, b, nkv, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    o, lse = flash_fwd(q, k, v, causal, scale)
    torch.cuda.synchronize()
    G.check_status()
    ro, rl = attention_ref(q, k, v, causal, scale, return_lse=True)
    torch.testing.assert_close(o.float(), ro.float(), atol=2e-2, rtol=2e-2)
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
