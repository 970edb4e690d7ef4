"""Exponent / mantissa split compression is bit-exact and actually shrinks activation-like data."""
import pytest
import torch

from mindspeed_b200.ops.compress import compress, decompress


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_bit_exact_roundtrip(dtype):
    torch.manual_seed(0)
    x = (torch.randn(3, 1000) * torch.logspace(-3, 3, 1000)).to(dtype)
    x[0, :5] = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan")]).to(dtype)
    x[1, 0] = torch.finfo(dtype).tiny / 4                      # a denormal
    c = compress(x)
    y = decompress(c)
    itype = torch.int16 if dtype != torch.float32 else torch.int32
    assert y.shape == x.shape and torch.equal(y.view(itype), x.view(itype))


def test_activation_like_data_compresses():
    torch.manual_seed(1)
    act = torch.nn.functional.gelu(torch.randn(64, 4096)).bfloat16()
    c = compress(act)
    assert c.ratio() < 0.85, c.ratio()                         # narrow exponent range per block: > 15 % smaller
    const = torch.full((4096,), 1.5, dtype=torch.bfloat16)
    assert compress(const).ratio() < 0.52                      # width 0: only sign + mantissa remain
    assert torch.equal(decompress(compress(const)), const)
