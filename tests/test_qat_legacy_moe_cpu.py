"""Fake-quant QAT, distillation loss, and the DeepSpeed-style MoE layer."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def test_fake_quantize_grid_and_ste():
    from mindspeed_b200.qat import fake_quantize
    x = torch.linspace(-1, 1, 256).view(2, 128).clone().requires_grad_(True)
    for bits in (4, 8):
        y = fake_quantize(x, bits, group=64)
        assert len(torch.unique(y[0, :64])) <= 2 ** bits
        assert (y - x).abs().max() <= 1.0 / (2 ** (bits - 1) - 1) / 2 + 1e-6
    y.sum().backward()
    assert torch.allclose(x.grad, torch.ones_like(x))          # straight-through inside the range
    ya = fake_quantize(x.detach(), 4, group=-1, symmetric=False)
    assert (ya - x.detach()).abs().max() <= 2.0 / 15 / 2 + 1e-6


def test_apply_qat_and_distill():
    from mindspeed_b200.qat import DistillConfig, QATConfig, TeacherManager, apply_qat, distillation_loss
    torch.manual_seed(0)
    teacher = nn.Sequential(nn.Linear(128, 256), nn.GELU(), nn.Linear(256, 64))
    student = nn.Sequential(nn.Linear(128, 256), nn.GELU(), nn.Linear(256, 64))
    student.load_state_dict(teacher.state_dict())
    assert apply_qat(student, QATConfig(scheme="W4A8", weight_group=64)) == 2
    tm = TeacherManager(teacher, DistillConfig(temperature=2.0))
    opt = torch.optim.Adam(student.parameters(), lr=1e-3)
    x = torch.randn(64, 128)
    first = None
    for _ in range(30):
        tl = tm.forward(x)
        loss = distillation_loss(student(x), tl, tm.cfg)
        first = first if first is not None else float(loss)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < first and float(loss) >= 0
    assert all(not p.requires_grad for p in teacher.parameters())
    # identical logits -> zero KL
    assert abs(float(distillation_loss(tl, tl, tm.cfg))) < 1e-6


def test_gating_capacity_and_aux():
    from mindspeed_b200.legacy_moe import top1gating, top2gating
    torch.manual_seed(1)
    logits = torch.randn(64, 4)
    l, comb, disp, cnt = top1gating(logits, capacity_factor=1.0, min_capacity=4)
    assert comb.shape == (64, 4, 16) and disp.sum() <= 64 and l > 0 and cnt.sum() == 64
    assert disp.sum(dim=(0,)).max() <= 1                       # one token per buffer slot
    l2, comb2, disp2, cnt2 = top2gating(logits, capacity_factor=1.0, min_capacity=4)
    assert comb2.shape == (64, 4, 32) and cnt2.sum() == 128
    kept = disp2.sum(dim=(1, 2))
    w = comb2.sum(dim=(1, 2))
    assert torch.allclose(w[kept == 2], torch.ones_like(w[kept == 2]), atol=1e-5)


def _moe_rank(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.legacy_moe import MoE
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(5)
    expert = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 16))
    full = MoE(16, expert, num_experts=4, ep_size=1, k=2, capacity_factor=4.0)
    torch.manual_seed(5)
    expert2 = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 16))
    par = MoE(16, expert2, num_experts=4, ep_size=world, k=2, capacity_factor=4.0, ep_group=dist.group.WORLD, pipe_experts=2)
    par.moe_layer.gate.load_state_dict(full.moe_layer.gate.state_dict())
    # give every global expert distinct weights, the same in both layers
    for e in range(4):
        g = torch.Generator().manual_seed(100 + e)
        for p in full.moe_layer.experts.experts[e].parameters():
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
    nl = 4 // world
    for le in range(nl):
        par.moe_layer.experts.experts[le].load_state_dict(full.moe_layer.experts.experts[rank * nl + le].state_dict())
    xs = [torch.randn(10, 16, generator=torch.Generator().manual_seed(7 + r)) for r in range(world)]
    out, aux, cnt = par(xs[rank])
    ref, _, _ = full(xs[rank])
    # capacity is generous, so no token is dropped and routing per rank is identical to the single-process layer
    ok = torch.allclose(out, ref, atol=1e-5)
    dist.destroy_process_group()
    return ok


def test_legacy_moe_expert_parallel_matches_local():
    assert all(run_distributed(_moe_rank, 2))


def _train_legacy(rank, world, prefix, extra):
    import io
    import os
    import sys
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    flags = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-model-type", "deepspeed_moe", "--moe-aux-loss-coeff", "0.01",
             "--expert-model-parallel-size", str(world), "--moe-no-drop", "--data-path", prefix, "--split", "100,0,0",
             "--train-iters", "8", "--lr", "1e-2"]
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + flags + list(extra))
    return [h["lm loss"] for h in hist]


def test_deepspeed_style_moe_trains_and_pipelined_experts_change_nothing(tmp_path):
    """--moe-model-type deepspeed_moe in the transformer layer: learns a small corpus; cutting the capacity dimension into
    chunks (--use-pipe-experts --pipe-experts-multi-data 2) is the same computation."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    from test_gpt_dataset_cpu import _corpus
    prefix = str(tmp_path / "c")
    _corpus(prefix, n_docs=60, vocab=100)
    plain = run_distributed(_train_legacy, 2, prefix, [])[0]
    piped = run_distributed(_train_legacy, 2, prefix, ["--use-pipe-experts", "--pipe-experts-multi-data", "2",
                                                       "--pipe-experts-multi-stream"])[0]
    assert plain[-1] < plain[0] - 0.1, plain
    for a, b in zip(plain, piped):
        assert abs(a - b) < 1e-5 * max(1.0, abs(a)), (plain, piped)


def test_ampipe_pipelines_the_moe_over_sequence_slices(tmp_path):
    """--ampipe-degree 2: residual add, norm and the DeepSpeed-style MoE behind the attention run on two sequence slices.
    With --moe-no-drop every slice routes as the whole sequence would, so the training run is the same."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    from test_gpt_dataset_cpu import _corpus
    prefix = str(tmp_path / "c")
    _corpus(prefix, n_docs=60, vocab=100)
    plain = run_distributed(_train_legacy, 2, prefix, ["--moe-aux-loss-coeff", "0.0", "--train-iters", "3"])[0]
    sliced = run_distributed(_train_legacy, 2, prefix, ["--moe-aux-loss-coeff", "0.0", "--train-iters", "3", "--ampipe-degree", "2"])[0]
    assert len(plain) == 3
    for a, b in zip(plain, sliced):
        assert abs(a - b) < 2e-5 * max(1.0, abs(a)), (plain, sliced)
    # the slices were in fact used
    from mindspeed_b200.config import TransformerConfig
    import torch
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True, optimization_level=0)
    cfg.ampipe_degree = 2
    from mindspeed_b200.models.transformer import TransformerLayer
    import torch.distributed as dist
    from mindspeed_b200.parallel import parallel_state as ps
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", str(__import__("dist_utils")._free_port()))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1, 1)
    assert TransformerLayer(cfg, 1).ampipe == 1                      # a dense layer ignores the option
    ps.destroy_model_parallel()
