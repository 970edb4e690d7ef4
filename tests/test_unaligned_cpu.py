import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def test_split_sizes():
    from mindspeed_b200.parallel.unaligned import split_sizes
    assert split_sizes(10, 3) == [4, 3, 3]
    assert split_sizes(5 * 16, 3, unit=16) == [32, 32, 16]          # 5 heads of 16 over 3 ranks


def _run(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.unaligned import UnalignedColumnParallelLinear, UnalignedRowParallelLinear, split_sizes
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(tensor_model_parallel_size=world)
    cfg = TransformerConfig(num_layers=1, hidden_size=20, num_attention_heads=5, unaligned_linear=True, use_cpu_initialization=True,
                            optimization_level=0) if False else None
    class C:  # minimal config: only what the layers read
        params_dtype = torch.float32
    g = torch.Generator().manual_seed(0)
    S, H, F = 10, 20, 35
    X = torch.randn(S, 2, H, generator=g)
    W1, W2 = torch.randn(F, H, generator=g) * 0.1, torch.randn(H, F, generator=g) * 0.1
    seq = split_sizes(S, world)
    col = UnalignedColumnParallelLinear(H, F, config=C, init_method=lambda t: t.copy_(W1), bias=False, sequence_parallel_sizes=seq)
    row = UnalignedRowParallelLinear(F, H, config=C, init_method=lambda t: t.copy_(W2), bias=False, sequence_parallel_sizes=seq)
    start = sum(seq[:rank])
    xl = X[start:start + seq[rank]].clone().requires_grad_(True)
    h, _ = col(xl)
    y, _ = row(torch.relu(h))
    y.sum().backward()
    Xr = X.clone().requires_grad_(True)
    ref = torch.relu(Xr @ W1.t()) @ W2.t()
    ref.sum().backward()
    out = {"y": (y.detach() - ref.detach()[start:start + seq[rank]]).abs().max().item(),
           "dx": (xl.grad - Xr.grad[start:start + seq[rank]]).abs().max().item()}
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return out


def test_unaligned_tp3_sequence_parallel_matches_dense():
    for r in run_distributed(_run, 3):
        assert r["y"] < 1e-5 and r["dx"] < 1e-5, r
