"""Fused reduce-scatter + AdamW + all-gather kernel against all-reduce + torch AdamW on >= 2 GPUs."""
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
        from mindspeed_b200.ops.fused_dist_opt import FusedShardedAdam
        grp = dist.new_group(list(range(world)))
        for grad_dtype, clip, tag in ((torch.float32, 0.0, "a"), (torch.bfloat16, 0.5, "b")):
            n = 1_000_003
            torch.manual_seed(0)
            w0 = (torch.randn(n, device="cuda") * 0.1).bfloat16()
            opt = FusedShardedAdam(grp, n, grad_dtype, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, tag=tag)
            opt.init_from_params(w0)
            ref_p = torch.nn.Parameter(w0.float().clone())
            ref = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
            for step in range(4):
                g = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 * step + rank)).to(grad_dtype)
                opt.zero_grad()
                opt.grad_buffer[:n].copy_(g)
                torch.cuda.synchronize()
                norm = opt.step(grad_scale=1.0 / world, clip_grad=clip)
                gs = g.float().clone()
                dist.all_reduce(gs, group=grp)
                gs /= world
                if clip:
                    gn = gs.norm()
                    gs *= torch.clamp(clip / (gn + 1e-6), max=1.0)
                    assert abs(float(norm) - float(gn)) < 1e-3 * float(gn)
                ref_p.grad = gs
                ref.step()
                torch.cuda.synchronize()
                G.check_status()
                got = opt.param_buffer[:n].float()
                want = ref_p.detach().bfloat16().float()
                # every rank must hold the complete, identical, updated bucket
                bad = (got - want).abs() > 2e-2 * want.abs().clamp_min(1e-2)
                assert bad.float().mean().item() < 1e-4, (step, grad_dtype, bad.float().mean().item())
                mine = slice(rank * opt.shard, min(n, (rank + 1) * opt.shard))
                assert torch.allclose(opt.master[:mine.stop - mine.start], ref_p.detach()[mine], atol=2e-5, rtol=1e-4)
        dist.barrier()
        torch.cuda.synchronize()
        from mindspeed_b200.parallel.symm_mem import destroy_heaps
        destroy_heaps()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        import traceback
        q.put((rank, "err", traceback.format_exc()))


def test_fused_step_matches_allreduce_adamw():
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
