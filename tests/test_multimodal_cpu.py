"""Multi-model rank layout with boundary exchange, and depth-parallel 3-D convolution, on gloo ranks."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _conv_rank(rank, world, kd, pd):
    import torch.distributed as dist
    from mindspeed_b200.parallel.multimodal import Conv3dDepthParallel
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    ref = nn.Conv3d(3, 4, (kd, 3, 3), stride=(1, 2, 1), padding=(pd, 1, 1))
    x = torch.randn(2, 3, 4 * world, 6, 5, requires_grad=True)
    y_ref = ref(x)
    gy = torch.randn_like(y_ref)
    y_ref.backward(gy)
    gx_ref, gw_ref = x.grad.clone(), ref.weight.grad.clone()
    ref.zero_grad()
    par = Conv3dDepthParallel(3, 4, (kd, 3, 3), group=dist.group.WORLD, conv=ref)
    xs = x.detach()[:, :, 4 * rank:4 * (rank + 1)].clone().requires_grad_(True)
    ys = par(xs)
    # output slabs: rank r owns outputs [4r, 4r + len)
    lens = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(lens, torch.tensor([ys.shape[2]]))
    start = sum(int(l) for l in lens[:rank])
    assert sum(int(l) for l in lens) == y_ref.shape[2]
    assert torch.allclose(ys, y_ref[:, :, start:start + ys.shape[2]], atol=1e-5)
    ys.backward(gy[:, :, start:start + ys.shape[2]])
    par.allreduce_weight_grads()
    assert torch.allclose(xs.grad, gx_ref[:, :, 4 * rank:4 * (rank + 1)], atol=1e-5)
    assert torch.allclose(ref.weight.grad, gw_ref, atol=1e-4)
    dist.destroy_process_group()
    return True


@pytest.mark.parametrize("world,kd,pd", [(2, 3, 1), (3, 3, 1), (2, 3, 0), (2, 4, 1)])
def test_conv3d_depth_parallel(world, kd, pd):
    assert all(run_distributed(_conv_rank, world, kd, pd))


class Enc(nn.Module):
    def __init__(self):
        super().__init__()
        self.l = nn.Linear(6, 8)

    def forward(self, x):
        return torch.tanh(self.l(x))


class Dec(nn.Module):
    def __init__(self):
        super().__init__()
        self.l = nn.Linear(8, 1)

    def forward(self, h, y):
        return ((self.l(h).squeeze(-1) - y) ** 2).mean()


def _data(n_mb):
    g = torch.Generator().manual_seed(9)
    return [(torch.randn(4, 6, generator=g), torch.randn(4, generator=g)) for _ in range(n_mb)]


def _dist_rank(rank, world, enc_world, dec_world, n_mb):
    import torch.distributed as dist
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel import multimodal as mm
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = mm.DistTrainConfig.from_list([dict(name="vit", world_size=enc_world), dict(name="gpt", world_size=dec_world, main_dp=True)])
    mm.initialize_dist_train(cfg)
    assert mm.get_dist_model_index() == (0 if rank < enc_world else 1)
    assert ps.get_data_parallel_world_size() == (enc_world if rank < enc_world else dec_world)
    assert ps.get_tensor_model_parallel_world_size() == 1
    torch.manual_seed(0)
    enc, dec = Enc(), Dec()
    data = _data(n_mb)
    out = {}
    if mm.is_in_model("vit"):
        # encoder ranks split every micro-batch's rows between them
        r, n = ps.get_data_parallel_rank(), enc_world
        per = 4 // n
        it = iter([(x[r * per:(r + 1) * per], None) for x, _ in data])
        mm.dist_forward_backward(lambda b, m, xin: m(b[0]), it, enc, n_mb)
        out["grad"] = enc.l.weight.grad.clone()
    else:
        r, n = ps.get_data_parallel_rank(), dec_world
        f = max(1, enc_world // dec_world)
        rows_per_dec = 4 // n if enc_world <= dec_world else 4 // dec_world
        # with fewer encoders than decoders every decoder sees the whole encoder output: it picks its rows of y
        def step(b, m, h):
            y = b[1]
            if enc_world <= dec_world:
                per_src = 4 // enc_world
                src = r // (dec_world // enc_world)
                y = y[src * per_src:(src + 1) * per_src]
            else:
                y = y[r * rows_per_dec:(r + 1) * rows_per_dec]
            return m(h, y)
        losses = mm.dist_forward_backward(step, iter(data), dec, n_mb)
        out["loss"] = torch.stack(losses)
        out["grad"] = dec.l.weight.grad.clone()
    dist.barrier()
    mm.destroy_dist_train()
    dist.destroy_process_group()
    return out


def test_two_models_on_disjoint_ranks_match_composed_model():
    n_mb = 2
    torch.manual_seed(0)
    enc, dec = Enc(), Dec()
    tot = 0
    for x, y in _data(n_mb):
        loss = dec(enc(x), y) / n_mb
        loss.backward()
    # 2 encoder ranks (each half of the rows) -> 1 decoder rank (concatenates): identical to the composed model
    res = run_distributed(_dist_rank, 3, 2, 1, n_mb)
    g_enc = sum(torch.as_tensor(r["grad"]) for r in res[:2])
    assert torch.allclose(g_enc, enc.l.weight.grad, atol=1e-5)
    assert torch.allclose(torch.as_tensor(res[2]["grad"]), dec.l.weight.grad, atol=1e-5)


def test_header_roundtrip_and_config_validation():
    from mindspeed_b200.parallel.multimodal import dist_train as D
    t = torch.zeros(2, 3, 5, dtype=torch.bfloat16, requires_grad=True)
    assert D.decode_header(D.encode_header(t)) == (torch.bfloat16, True, (2, 3, 5))
    assert D.decode_header(D.encode_header(None)) is None
    with pytest.raises(ValueError):
        D.DistTrainConfig.from_list([dict(name="a", world_size=3, tensor_model_parallel_size=2)]).validate(3)
    with pytest.raises(ValueError):
        D.DistTrainConfig.from_list([dict(name="a", world_size=2), dict(name="b", world_size=2)]).validate(5)
    assert D._peers([0, 1], [2, 3, 4, 5], 1, True) == [4, 5] and D._peers([0, 1], [2, 3, 4, 5], 3, False) == [0]
    assert D._peers([0, 1, 2, 3], [4, 5], 2, True) == [5] and D._peers([0, 1, 2, 3], [4, 5], 4, False) == [0, 1]
