import torch


def test_split_merge_roundtrip_cpu():
    from mindspeed_b200.memory.reuse_param import adam_flat_reuse, merge_fp32, split_fp32
    torch.manual_seed(0)
    p = torch.cat([torch.randn(5000) * 10 ** torch.randint(-6, 6, (5000,)).float(), torch.tensor([0.0, -0.0, 1.0, -1.0])])
    hi, lo = split_fp32(p)
    assert hi.dtype == torch.bfloat16 and lo.dtype == torch.int16
    assert torch.equal(merge_fp32(hi, lo), p)
    # hi is within half a bf16 ulp of the master
    assert ((hi.float() - p).abs() <= p.abs() * 2 ** -8 + 1e-30).all()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    ref, m2, v2 = p.clone(), torch.zeros_like(p), torch.zeros_like(p)
    from mindspeed_b200.ops.adam import adam_flat_ref
    g = torch.randn_like(p)
    adam_flat_reuse(hi, lo, g, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.0, 1)
    adam_flat_ref(ref, g, m2, v2, None, 1e-3, 0.9, 0.95, 1e-8, 0.0, 1)
    torch.testing.assert_close(merge_fp32(hi, lo), ref)
