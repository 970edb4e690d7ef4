"""2-D tensor parallel linear and norms on 4 gloo ranks (x=2, y=2) against the dense computation."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _run(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.tp2d import ParallelLinear2D, RMSNorm2D
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(tensor_model_parallel_size=4, tp_2d=True, tp_x=2, tp_y=2)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True, optimization_level=0)
    gx, gy = ps.get_tp_x_group(), ps.get_tp_y_group()
    xi, yi = ps.get_tp_x_rank(), ps.get_tp_y_rank()
    S, B, H, E = 16, 2, 32, 48
    g = torch.Generator().manual_seed(0)
    X = torch.randn(S, B, H, generator=g)
    W1 = torch.randn(E, H, generator=g) * 0.1
    W2 = torch.randn(H, E, generator=g) * 0.1
    Wgt = torch.randn(S, B, H, generator=g)

    def init(w):
        return lambda t: t.copy_(w)
    l1 = ParallelLinear2D(H, E, config=cfg, init_method=init(W1), ag_group=gx, rs_group=gy)   # seq over x, hidden over y
    l2 = ParallelLinear2D(E, H, config=cfg, init_method=init(W2), ag_group=gy, rs_group=gx)   # roles swapped
    norm = RMSNorm2D(H, 1e-5, cfg, group=gy)
    xl = X.chunk(2, 0)[xi].chunk(2, 2)[yi].clone().requires_grad_(True)
    h, _ = l1(norm(xl))
    out, _ = l2(torch.tanh(h))
    wl = Wgt.chunk(2, 0)[xi].chunk(2, 2)[yi]
    (out * wl).sum().backward()
    # dense reference
    Xr = X.clone().requires_grad_(True)
    W1r, W2r = W1.clone().requires_grad_(True), W2.clone().requires_grad_(True)
    nr = Xr * torch.rsqrt(Xr.pow(2).mean(-1, keepdim=True) + 1e-5)
    ref = torch.tanh(nr @ W1r.t()) @ W2r.t()
    (ref * Wgt).sum().backward()
    res = {"out": (out.detach() - ref.detach().chunk(2, 0)[xi].chunk(2, 2)[yi]).abs().max().item(),
           "dx": (xl.grad - Xr.grad.chunk(2, 0)[xi].chunk(2, 2)[yi]).abs().max().item(),
           "dw1": (l1.weight.grad - W1r.grad.chunk(2, 0)[xi].chunk(2, 1)[yi]).abs().max().item(),
           "dw2": (l2.weight.grad - W2r.grad.chunk(2, 0)[yi].chunk(2, 1)[xi]).abs().max().item()}
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return res


def test_tp2d_linear_and_norm_match_dense():
    for r in run_distributed(_run, 4):
        for k, v in r.items():
            assert v < 1e-4, (k, v, r)
