"""Staged MoE layer + forward/backward interleaving: same outputs and gradients as plain autograd."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _config(ep, shared):
    import torch.nn.functional as F
    from mindspeed_b200.config import TransformerConfig
    return TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, num_moe_experts=4,
                             moe_router_topk=2, moe_ffn_hidden_size=48, moe_grouped_gemm=True, gated_linear_unit=True,
                             activation_func=F.silu, add_bias_linear=False, expert_model_parallel_size=ep,
                             moe_token_dispatcher_type="alltoall", moe_aux_loss_coeff=0.01, use_cpu_initialization=True,
                             moe_shared_expert_intermediate_size=32 if shared else None, optimization_level=0,
                             hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm")


def _run(rank, world, shared):
    import torch.distributed as dist
    from mindspeed_b200.models.transformer import TransformerLayer
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.moe import fb_overlap as FB
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(expert_model_parallel_size=world)
    torch.manual_seed(3)
    cfg = _config(world, shared)
    layers = [TransformerLayer(cfg, layer_number=i + 1, is_moe=True) for i in range(2)]
    for l in layers:
        l.train()
    g = torch.Generator().manual_seed(100 + rank)
    xs = [torch.randn(6, 2, 32, generator=g) for _ in range(3)]
    ws = [torch.randn(6, 2, 32, generator=g) for _ in range(3)]

    # reference: ordinary autograd, micro-batch after micro-batch
    ref_out, ref_gin = [], []
    for x, w in zip(xs, ws):
        xi = x.clone().requires_grad_(True)
        h = xi
        for l in layers:
            h, _ = l(h)
        (h * w).sum().backward()
        ref_out.append(h.detach())
        ref_gin.append(xi.grad.clone())
    ref_pg = {n: p.grad.clone() for l_i, l in enumerate(layers) for n, p in l.named_parameters(prefix=str(l_i)) if p.grad is not None}
    for l in layers:
        l.zero_grad(set_to_none=True)

    outs, gins = FB.run_microbatches_overlapped(layers, xs, lambda i, out: ws[i])
    for a, b in zip(outs, ref_out):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    for a, b in zip(gins, ref_gin):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    for l_i, l in enumerate(layers):
        for n, p in l.named_parameters(prefix=str(l_i)):
            if n in ref_pg:
                assert p.grad is not None and torch.allclose(p.grad, ref_pg[n], atol=1e-4), n
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return True


@pytest.mark.parametrize("world,shared", [(1, False), (2, True)])
def test_overlapped_equals_sequential(world, shared):
    assert all(run_distributed(_run, world, shared))


def test_layer_graph_stage_bookkeeping():
    from mindspeed_b200.parallel.moe.fb_overlap import LayerGraph
    g = LayerGraph()
    x = torch.randn(3, requires_grad=True)
    a, b = g.run_stage(lambda t: (t * 2, t + 1), (x,))
    (c,) = g.run_stage(lambda u, v: u * v, (a, b))
    assert g.stages_left == 2 and not c.requires_grad
    ga, gb = g.backward_stage((torch.ones(3),))
    (gx,) = g.backward_stage((ga, gb))
    assert g.stages_left == 0
    assert torch.allclose(gx, 2 * (x.detach() + 1) + 2 * x.detach())


def _train_losses(rank, world, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import io
    from contextlib import redirect_stdout
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    moe = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-token-dispatcher-type", "alltoall", "--moe-grouped-gemm",
           "--moe-aux-loss-coeff", "0.01", "--expert-model-parallel-size", str(world), "--use-distributed-optimizer"]
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + moe + list(extra))
    return [h["lm loss"] for h in hist]


@pytest.mark.parametrize("world", [1, 2])
def test_training_with_fb_overlap_matches_plain_schedule(world):
    """``--moe-fb-overlap`` (micro-batch i's forward interleaved with micro-batch i-1's backward inside the layer stack)
    gives the same losses as the plain schedule, with expert parallelism and the distributed optimizer."""
    ref = run_distributed(_train_losses, world, [])[0]
    got = run_distributed(_train_losses, world, ["--moe-fb-overlap"])[0]
    assert len(ref) == 3
    for a, b in zip(ref, got):
        assert abs(a - b) < 1e-5 * max(1.0, abs(a)), (ref, got)


def test_training_with_hot_expert_replicas_matches_plain_dispatch():
    """``--balanced-moe-experts``: after the first step the busiest experts are replicated on both expert-parallel ranks and
    their tokens are computed locally; outputs and gradients (returned to the owner) are those of the plain dispatch."""
    ref = run_distributed(_train_losses, 2, [])[0]
    got = run_distributed(_train_losses, 2, ["--balanced-moe-experts", "--balanced-moe-hot-expert-num", "2",
                                             "--trans-hot-expert-group-num", "2"])[0]
    for a, b in zip(ref, got):
        assert abs(a - b) < 1e-5 * max(1.0, abs(a)), (ref, got)


def _train_pp(rank, world, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import io
    from contextlib import redirect_stdout
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    moe = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-token-dispatcher-type", "alltoall", "--moe-grouped-gemm",
           "--moe-aux-loss-coeff", "0.01", "--expert-model-parallel-size", "2", "--pipeline-model-parallel-size", "2"]
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + moe + list(extra))
    return [h.get("lm loss") for h in hist]


@pytest.mark.parametrize("schedule", [[], ["--num-layers-per-virtual-pipeline-stage", "1"], ["--schedules-method", "dualpipev"],
                                      # a no-op layer (identity, used to balance stages) inside the overlapped chunks
                                      ["--schedules-method", "dualpipev", "--noop-layers", "1"]])
def test_pipeline_schedules_with_fb_overlap_match_plain(schedule):
    """Pipeline 2 x expert parallel 2 on four ranks: with ``--moe-fb-overlap`` the schedules put an F and a B of different
    micro-batches into one slot and interleave them stage by stage; the losses are those of the unpaired schedule."""
    ref = run_distributed(_train_pp, 4, schedule)
    got = run_distributed(_train_pp, 4, schedule + ["--moe-fb-overlap"])
    ref_l = [r for r in ref if r[0] is not None][0]
    got_l = [r for r in got if r[0] is not None][0]
    assert len(ref_l) == 3
    for a, b in zip(ref_l, got_l):
        assert abs(a - b) < 1e-5 * max(1.0, abs(a)), (ref_l, got_l)


def test_paired_plans_are_valid():
    from mindspeed_b200.parallel.pipeline.plan import build_plan, validate
    for name, vpp in (("1f1b", None), ("interleaved", 2), ("dualpipev", None)):
        for pp in (2, 4):
            plain, paired = build_plan(name, pp, 8, vpp=vpp), build_plan(name, pp, 8, vpp=vpp, pair_fb=True)
            validate(paired)
            assert paired.num_slots < plain.num_slots
            assert any({o.kind for o in slot} >= {"F", "B"} for r in range(pp) for slot in paired.table[r])
            for r in range(pp):      # a pair never holds the forward and the backward of one micro-batch of one chunk
                for slot in paired.table[r]:
                    fs = {(o.chunk, o.mb) for o in slot if o.kind == "F"}
                    bs = {(o.chunk, o.mb) for o in slot if o.kind == "B"}
                    assert not (fs & bs) and len(fs) <= 1 and len(bs) <= 1
