"""MoE layer on CPU/gloo: expert-parallel all-to-all and all-gather dispatchers against the single-rank layer."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _make_config(ep, dispatcher, grouped=True, shared=False, score="softmax"):
    import torch.nn.functional as F
    from mindspeed_b200.config import TransformerConfig
    overlap_gather = dispatcher == "allgather_overlap"
    dispatcher = "allgather" if overlap_gather else dispatcher
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, num_moe_experts=4,
                             moe_router_topk=2, moe_ffn_hidden_size=96, moe_grouped_gemm=grouped, gated_linear_unit=True,
                             activation_func=F.silu, add_bias_linear=False, expert_model_parallel_size=ep,
                             moe_token_dispatcher_type=dispatcher, moe_aux_loss_coeff=0.01, use_cpu_initialization=True,
                             moe_shared_expert_intermediate_size=64 if shared else None, optimization_level=0,
                             moe_router_score_function=score, hidden_dropout=0.0, attention_dropout=0.0)
    cfg.moe_allgather_overlap_comm = overlap_gather     # all-gather of the hidden states started before the router
    return cfg


def _set_weights(layer, local_experts):
    g = torch.Generator().manual_seed(99)
    E, H, Fh = 4, 64, 96
    w1 = torch.randn(E, H, 2 * Fh, generator=g) * 0.05
    w2 = torch.randn(E, Fh, H, generator=g) * 0.05
    rw = torch.randn(E, H, generator=g) * 0.2
    with torch.no_grad():
        layer.router.weight.copy_(rw)
        if hasattr(layer.experts, "weight1"):
            layer.experts.weight1.copy_(w1[local_experts])
            layer.experts.weight2.copy_(w2[local_experts])
        else:
            for i, e in enumerate(local_experts):
                layer.experts.local_experts[i].linear_fc1.weight.copy_(w1[e].t())
                layer.experts.local_experts[i].linear_fc2.weight.copy_(w2[e].t())
        if layer.shared_experts is not None:
            sg = torch.Generator().manual_seed(5)
            layer.shared_experts.linear_fc1.weight.copy_(torch.randn(layer.shared_experts.linear_fc1.weight.shape, generator=sg) * 0.05)
            layer.shared_experts.linear_fc2.weight.copy_(torch.randn(layer.shared_experts.linear_fc2.weight.shape, generator=sg) * 0.05)


def _run(rank, world, ep, dispatcher, grouped, shared, score):
    import torch.distributed as dist
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.moe import MoELayer
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(expert_model_parallel_size=ep)
    cfg = _make_config(ep, dispatcher, grouped, shared, score)
    layer = MoELayer(cfg, layer_number=1)
    _set_weights(layer, layer.local_expert_indices)
    layer.train()
    outs = []
    for dp_rank in range(2):           # the data both ranks of the EP=2 run see
        gx = torch.Generator().manual_seed(1000 + dp_rank)
        x = torch.randn(16, 2, 64, generator=gx)
        if world == 2 and dp_rank != rank:
            continue
        x.requires_grad_(True)
        y, _ = layer(x)
        loss = (y * torch.linspace(0, 1, 64)).sum()
        loss.backward()
        outs.append((dp_rank, y.detach().clone(), x.grad.clone()))
    grads = {}
    if hasattr(layer.experts, "weight1"):
        g1 = layer.experts.weight1.grad
        for i, e in enumerate(layer.local_expert_indices):
            grads[e] = g1[i].clone()
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return outs, grads


@pytest.mark.parametrize("dispatcher,grouped,shared,score", [("alltoall", True, False, "softmax"), ("alltoall", False, True, "sigmoid"),
                                                            ("allgather", True, False, "softmax"),
                                                            ("allgather_overlap", True, True, "softmax")])
def test_expert_parallel_matches_single_rank(dispatcher, grouped, shared, score):
    ref_outs, ref_grads = run_distributed(_run, 1, 1, dispatcher, grouped, shared, score)[0]
    res = run_distributed(_run, 2, 2, dispatcher, grouped, shared, score)
    for r in range(2):
        outs, grads = res[r]
        (dp, y, gx) = outs[0]
        t = torch.as_tensor
        yr, gxr = ref_outs[dp][1], ref_outs[dp][2]
        torch.testing.assert_close(t(y), t(yr), atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(t(gx), t(gxr), atol=1e-5, rtol=1e-4)
        for e, g in grads.items():
            # single-rank reference accumulated both data shards into one grad
            torch.testing.assert_close(t(g), t(ref_grads[e]), atol=1e-5, rtol=1e-4)


def test_permute_unpermute_roundtrip():
    from mindspeed_b200.parallel.moe.moe_utils import permute, unpermute, topk_softmax_with_capacity
    torch.manual_seed(0)
    x = torch.randn(10, 8)
    logits = torch.randn(10, 4)
    probs, rmap, tpe = topk_softmax_with_capacity(logits, 2)
    assert rmap.sum().item() == 20 and tpe.sum().item() == 20
    p, idx = permute(x, rmap)
    back = unpermute(p, idx, x.shape, probs, rmap)
    torch.testing.assert_close(back, x * probs.sum(1, keepdim=True))
