"""Peer-memory Ulysses all-to-alls (layout transform fused in) against the NCCL + permute path, values and gradients."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world)
        from mindspeed_b200.ops import gemm as G
        from mindspeed_b200.parallel.context_parallel import ulysses as U
        grp = dist.new_group(list(range(world)))
        for dtype, (sl, b, n, d) in ((torch.bfloat16, (64, 2, 8, 128)), (torch.float32, (33, 1, 4 * world, 64))):
            for it in range(3):                                   # repeated calls recycle the two staging slots
                torch.manual_seed(10 * it + rank)
                x = torch.randn(sl, b, n, d, device="cuda").to(dtype)
                xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
                U.set_fused_all_to_all(False)
                ya = U.seq_to_heads(xa, grp)
                za = U.heads_to_seq(ya * 2.0, grp)
                U.set_fused_all_to_all(True)
                yb = U.seq_to_heads(xb, grp)
                zb = U.heads_to_seq(yb * 2.0, grp)
                torch.cuda.synchronize()
                G.check_status()
                assert ya.shape == yb.shape == (sl * world, b, n // world, d)
                assert torch.equal(ya, yb) and torch.equal(za, zb)
                assert torch.equal(za, x * 2.0)                    # the round trip is the identity
                g = torch.randn_like(za)
                za.backward(g)
                zb.backward(g)
                torch.cuda.synchronize()
                G.check_status()
                assert torch.equal(xa.grad, xb.grad)
        U.set_fused_all_to_all(False)
        dist.barrier()
        torch.cuda.synchronize()
        from mindspeed_b200.parallel.symm_mem import destroy_heaps
        destroy_heaps()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        import traceback
        q.put((rank, "err", traceback.format_exc()))


def test_fused_ulysses_all_to_all_matches_nccl():
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in range(world):
            out.append(q.get(timeout=240))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    bad = [o for o in out if o[1] != "ok"]
    assert not bad, bad[0][2]
