"""Peer-memory MoE dispatch / combine against the NCCL all-to-all dispatcher on the same routing (>= 2 GPUs)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _config(ep, fused):
    import torch.nn.functional as F
    from mindspeed_b200.config import TransformerConfig
    cfg = TransformerConfig(num_layers=2, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, num_moe_experts=8,
                             moe_router_topk=2, moe_ffn_hidden_size=256, moe_grouped_gemm=True, gated_linear_unit=True,
                             activation_func=F.silu, add_bias_linear=False, expert_model_parallel_size=ep,
                             moe_token_dispatcher_type="alltoall", moe_aux_loss_coeff=0.0, optimization_level=2,
                             params_dtype=torch.bfloat16, bf16=True, hidden_dropout=0.0, attention_dropout=0.0)
    cfg.moe_alltoall_mc2 = fused          # feature flag carried as an extra attribute, as update_from_args does
    return cfg


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world)
        from mindspeed_b200.ops import gemm as G
        from mindspeed_b200.parallel import parallel_state as ps
        from mindspeed_b200.parallel.moe import MoELayer
        from mindspeed_b200.parallel.moe.fused_dispatcher import FusedAlltoAllTokenDispatcher
        ps.initialize_model_parallel(expert_model_parallel_size=world)
        torch.manual_seed(11)
        ref = MoELayer(_config(world, False), layer_number=1).cuda()
        fus = MoELayer(_config(world, True), layer_number=1).cuda()
        assert isinstance(fus.token_dispatcher, FusedAlltoAllTokenDispatcher)
        fus.load_state_dict(ref.state_dict())
        ref.train(); fus.train()
        # 1) dispatcher level: same rows in the same order, same probabilities
        for it in range(3):                         # repeated calls recycle the two staging slots
            torch.manual_seed(1000 * it + rank)
            x = (torch.randn(96, 2, 256, device="cuda") * 0.5).bfloat16()
            xr, xf = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            probs, rmap = ref.router(xr)
            probs = probs.to(x.dtype)
            rows_r, tpe_r, pr_r = ref.token_dispatcher.token_permutation(xr, probs, rmap)
            rows_f, tpe_f, pr_f = fus.token_dispatcher.token_permutation(xf, probs.detach().clone(), rmap)
            torch.cuda.synchronize()
            G.check_status()
            assert torch.equal(torch.as_tensor(tpe_r), torch.as_tensor(tpe_f))
            assert torch.equal(rows_r, rows_f), "dispatched rows differ"
            assert torch.equal(pr_r, pr_f), "dispatched probabilities differ"
            w = torch.linspace(0.5, 1.5, rows_r.shape[0], device="cuda").unsqueeze(-1).bfloat16()
            out_r, _ = ref.token_dispatcher.token_unpermutation(rows_r * w)
            out_f, _ = fus.token_dispatcher.token_unpermutation(rows_f * w)
            torch.cuda.synchronize()
            G.check_status()
            err = (out_r.float() - out_f.float()).abs().max().item()
            assert err <= 2e-2 * out_r.float().abs().max().item() + 1e-6, ("combine", err)
        # 2) layer level: outputs and gradients of the whole MoE layer
        for it in range(2):
            torch.manual_seed(77 + 10 * it + rank)
            x = (torch.randn(64, 2, 256, device="cuda") * 0.5).bfloat16()
            xr, xf = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            yr, _ = ref(xr)
            yf, _ = fus(xf)
            g = torch.randn_like(yr)
            yr.backward(g)
            yf.backward(g)
            torch.cuda.synchronize()
            G.check_status()

            def close(a, b, what, tol=3e-2):
                e = (a.float() - b.float()).abs().max().item()
                s = a.float().abs().max().item()
                assert e <= tol * s + 1e-5, (what, e, s)
            close(yr, yf, "output")
            close(xr.grad, xf.grad, "input grad")
            close(ref.router.weight.grad, fus.router.weight.grad, "router grad", 5e-2)
            close(ref.experts.weight1.grad, fus.experts.weight1.grad, "w1 grad")
            close(ref.experts.weight2.grad, fus.experts.weight2.grad, "w2 grad")
            for m in (ref, fus):
                m.zero_grad(set_to_none=True)
        assert fus.token_dispatcher.fused_calls >= 5 and fus.token_dispatcher.fallback_calls == 0
        # run-to-run determinism of the fused path
        torch.manual_seed(5 + rank)
        x = (torch.randn(64, 2, 256, device="cuda") * 0.5).bfloat16()
        with torch.no_grad():
            y1, _ = fus(x)
            y2, _ = fus(x)
        assert torch.equal(y1, y2)
        dist.barrier()
        torch.cuda.synchronize()
        from mindspeed_b200.parallel.symm_mem import destroy_heaps
        destroy_heaps()
        ps.destroy_model_parallel()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        import traceback
        q.put((rank, "err", traceback.format_exc()))


def test_fused_dispatch_combine_match_all_to_all():
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
