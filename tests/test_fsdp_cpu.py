"""Fully sharded data parallel / hybrid sharding / LayerZeRO on gloo ranks against a single-process reference."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


class Block(nn.Module):
    def __init__(self, h):
        super().__init__()
        self.fc1, self.fc2, self.norm = nn.Linear(h, 3 * h), nn.Linear(3 * h, h), nn.LayerNorm(h)

    def forward(self, x):
        return x + self.fc2(torch.tanh(self.fc1(self.norm(x))))


class Net(nn.Module):
    def __init__(self, h=20, n=3):
        super().__init__()
        self.inp = nn.Linear(7, h)
        self.blocks = nn.ModuleList([Block(h) for _ in range(n)])
        self.out = nn.Linear(h, 5)
        self.unused = nn.Parameter(torch.ones(3))       # never touched by forward

    def forward(self, x):
        x = self.inp(x)
        for b in self.blocks:
            x = b(x)
        return self.out(x)


def _data(world, steps, mbs=2):
    g = torch.Generator().manual_seed(3)
    return [[[(torch.randn(4, 7, generator=g), torch.randn(4, 5, generator=g)) for _ in range(mbs)] for _ in range(world)]
            for _ in range(steps)]


def _reference(world, steps):
    torch.manual_seed(0)
    net = Net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, weight_decay=0.01)
    losses = []
    for step_data in _data(world, steps):
        opt.zero_grad()
        tot = 0.0
        for r in range(world):
            for x, y in step_data[r]:
                loss = ((net(x) - y) ** 2).mean() / (world * len(step_data[r]))
                loss.backward()
                tot += float(loss)
        net.unused.grad = None
        opt.step()
        losses.append(tot)
    return losses, {k: v.detach().clone() for k, v in net.state_dict().items()}


def _rank(rank, world, steps, shard_size, zero1, ignore=()):
    import torch.distributed as dist
    from mindspeed_b200.parallel.distributed.fsdp import FSDPPlan, fully_shard
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    net = Net()
    plan = FSDPPlan(wrap=["Block"], shard_size=shard_size, zero1_over_replicas=zero1, ignore=tuple(ignore))
    model = fully_shard(net, plan)
    assert len(model.units) == 4                       # three blocks + root
    if ignore:
        assert len(model.ignored) == 2 and all(p.numel() > 0 for p in model.ignored)       # out.weight, out.bias stay whole
    ms = model.memory_summary()
    assert ms["param_shard_bytes"] * (shard_size or world) >= ms["unsharded_bytes"]
    opt = torch.optim.AdamW(model.optimizer_params(), lr=1e-2, weight_decay=0.01)
    losses = []
    for step_data in _data(world, steps):
        model.zero_grad()
        tot = torch.zeros(())
        for x, y in step_data[rank]:
            loss = ((model(x) - y) ** 2).mean() / len(step_data[rank])
            loss.backward()
            tot += loss.detach()
        model.finish_grad_sync()
        opt.step()
        model.post_step()
        dist.all_reduce(tot)
        losses.append(float(tot) / world)
        assert all(p.numel() == 0 for u in model.units for p in u.params), "parameters must be resharded between steps"
    sd = model.full_state_dict()
    dist.destroy_process_group()
    return losses, sd


@pytest.mark.parametrize("world,shard_size,zero1", [(2, None, False), (4, 2, False), (4, 2, True)])
def test_sharded_training_matches_reference(world, shard_size, zero1):
    steps = 3
    ref_losses, ref_sd = _reference(world, steps)
    res = run_distributed(_rank, world, steps, shard_size, zero1)
    for losses, sd in res:
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 1e-5 * max(1.0, abs(b)), (losses, ref_losses)
        for k, v in ref_sd.items():
            if k == "unused":
                continue
            assert torch.allclose(torch.as_tensor(sd[k]), v, atol=2e-5, rtol=1e-4), k


def test_ignored_modules_stay_whole_and_train_the_same():
    """``FSDPPlan.ignore``: the output layer is not sharded; its gradients are averaged over the ranks instead."""
    steps = 3
    ref_losses, ref_sd = _reference(2, steps)
    for losses, sd in run_distributed(_rank, 2, steps, None, False, ["out"]):
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 1e-5 * max(1.0, abs(b)), (losses, ref_losses)
        for k in ("out.weight", "out.bias", "inp.weight", "blocks.1.fc.weight"):
            if k in ref_sd:
                assert torch.allclose(torch.as_tensor(sd[k]), ref_sd[k], atol=2e-5, rtol=1e-4), k


def test_plan_from_dict_and_yaml(tmp_path):
    from mindspeed_b200.parallel.distributed.fsdp import FSDPPlan
    p = FSDPPlan.from_dict({"fsdp": {"wrap": "blocks.*", "shard_size": 4, "param_dtype": "bfloat16"}})
    assert p.wrap == ["blocks.*"] and p.shard_size == 4 and p.param_dtype == "bfloat16"
    with pytest.raises(ValueError):
        FSDPPlan.from_dict({"nonsense": 1})
    f = tmp_path / "plan.yaml"
    f.write_text("fsdp:\n  wrap: [Block]\n  zero1_over_replicas: true\n")
    assert FSDPPlan.from_yaml(str(f)).zero1_over_replicas is True
