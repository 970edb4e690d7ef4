"""EP all-to-all + TP all-gather + BMM and its mirror, on 4 gloo ranks (ep 2 x tp 2), against a dense evaluation."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

E, C, H, Mh = 4, 3, 8, 12


def _rank(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.ops import moe_bmm_comm as B
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ep, tp = 2, 2
    tp_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    ep_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    ep_rank, tp_rank = rank // tp, rank % tp
    g_tp, g_ep = tp_groups[ep_rank], ep_groups[tp_rank]
    gen = torch.Generator().manual_seed(0)
    w1 = torch.randn(E, H, Mh, generator=gen)              # full expert weights
    w2 = torch.randn(E, Mh, H, generator=gen)
    xs = [torch.randn(E, C, H, generator=torch.Generator().manual_seed(10 + r)) for r in range(world)]
    e_loc, m_loc = E // ep, Mh // tp
    my_w1 = w1[ep_rank * e_loc:(ep_rank + 1) * e_loc, :, tp_rank * m_loc:(tp_rank + 1) * m_loc].contiguous().requires_grad_(True)
    my_w2 = w2[ep_rank * e_loc:(ep_rank + 1) * e_loc, tp_rank * m_loc:(tp_rank + 1) * m_loc, :].contiguous()
    x = xs[rank].clone().requires_grad_(True)
    h = B.all_to_all_all_gather_bmm(x, my_w1, g_ep, g_tp, shard_type=1, act_type="silu")
    assert h.shape == (e_loc, ep * C * tp, m_loc)
    y = B.bmm_reduce_scatter_all_to_all(h, my_w2, g_ep, g_tp, shard_type=1)
    assert y.shape == (E, C, H)
    # dense reference for this rank's tokens: y[e] = silu(x[e] @ w1[e]) @ w2[e]
    ref = torch.stack([torch.nn.functional.silu(xs[rank][e] @ w1[e]) @ w2[e] for e in range(E)])
    ok = torch.allclose(y, ref, atol=1e-4)
    y.sum().backward()
    ok = ok and x.grad is not None and my_w1.grad is not None and torch.isfinite(x.grad).all()
    # grouped matmul + all-reduce over tp
    rows = torch.randn(7, 6, generator=torch.Generator().manual_seed(3))
    wfull = [torch.randn(6, 5, generator=torch.Generator().manual_seed(20 + g)) for g in range(2)]
    k = 6 // tp
    out = B.grouped_matmul_all_reduce(rows[:, tp_rank * k:(tp_rank + 1) * k].contiguous(), [w[tp_rank * k:(tp_rank + 1) * k] for w in wfull],
                                      [3, 4], g_tp)
    refg = torch.cat([rows[:3] @ wfull[0], rows[3:] @ wfull[1]])
    ok = ok and torch.allclose(out, refg, atol=1e-4)
    dist.destroy_process_group()
    return bool(ok)


def test_bmm_comm_pair_matches_dense():
    assert all(run_distributed(_rank, 4))
