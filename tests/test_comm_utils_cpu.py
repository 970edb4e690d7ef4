"""Communication helpers on CPU/gloo ranks: side-stream API shape, buffer-size spec, sliced gather/scatter, delayed log all-reduce."""
import os
import sys
from types import SimpleNamespace

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def test_buffer_spec_and_auto_sizes():
    from mindspeed_b200.parallel import comm_utils as C
    assert C.parse_buffer_spec("dp:200; tp:64") == {"dp": 200, "tp": 64}
    with pytest.raises(ValueError):
        C.parse_buffer_spec("bogus:1")
    with pytest.raises(ValueError):
        C.parse_buffer_spec("dp")
    args = SimpleNamespace(seq_length=8192, context_parallel_size=1, micro_batch_size=1, hidden_size=4096,
                           tensor_model_parallel_size=8, num_attention_heads=32, num_query_groups=8, kv_channels=128,
                           sequence_parallel=True, num_experts=None, ddp_bucket_size=None,
                           hccl_group_buffer="tp:100", hccl_group_buffer_adaptive=True)
    sizes = C.auto_buffer_sizes(args)
    assert sizes["tp"] == 64 and sizes["pp"] == 8 and sizes["dp"] == 153
    opts = C.group_options(args)
    assert opts["tp"].buffer_mb == 100 and opts["tp"].max_ctas == 16 and opts["dp"].max_ctas is None


def _ranks(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.parallel import comm_utils as C
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = dist.group.WORLD
    # async helpers degrade to synchronous collectives on CPU but keep the (input, output, handle) contract
    x = torch.full((4, 3), float(rank + 1))
    _, ag, h = C.async_all_gather(x, g)
    h.wait()
    assert ag.shape == (4 * world, 3) and ag[4 * (world - 1)].eq(world).all()
    _, rs, h = C.async_reduce_scatter(torch.ones(4 * world, 2) * (rank + 1), g)
    h.wait()
    assert rs.shape == (4, 2) and rs.eq(sum(range(1, world + 1))).all()
    _, a2a, h = C.async_all_to_all(torch.arange(world * 2, dtype=torch.float32) + 100 * rank, None, None, g)
    h.wait()
    assert a2a.tolist() == [100 * r + 2 * rank + j for r in range(world) for j in range(2)]
    # sliced gather / scatter with a slice much smaller than the tensor
    local = torch.arange(1000, dtype=torch.float32).view(10, 100) + 10000 * rank
    parts = C.gather_to_rank0_sliced(local, g, slice_bytes=256)
    if rank == 0:
        assert all(torch.equal(parts[r], torch.arange(1000, dtype=torch.float32).view(10, 100) + 10000 * r) for r in range(world))
    back = C.scatter_from_rank0_sliced(parts, local, g, slice_bytes=256)
    assert torch.equal(back, local)
    # delayed logging all-reduce: results arrive one call late
    lg = C.AsyncLogAllReduce(g)
    assert lg.submit({"loss": torch.tensor(float(rank))}, step=1) is None
    step, vals = lg.submit({"loss": torch.tensor(float(rank) + 10)}, step=2)
    assert step == 1 and abs(vals["loss"] - (world - 1) / 2) < 1e-6
    step, vals = lg.flush()
    assert step == 2 and abs(vals["loss"] - (10 + (world - 1) / 2)) < 1e-6
    assert lg.flush() is None
    dist.destroy_process_group()
    return True


def test_helpers_on_gloo_ranks():
    assert all(run_distributed(_ranks, 2))
