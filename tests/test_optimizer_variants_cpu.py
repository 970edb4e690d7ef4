"""Optimizer variants through the full training loop on CPU (1 rank, gloo)."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

ARGS = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--ffn-hidden-size", "128", "--seq-length", "32",
        "--max-position-embeddings", "32", "--micro-batch-size", "2", "--global-batch-size", "4", "--vocab-size", "128",
        "--make-vocab-size-divisible-by", "1", "--lr", "1e-3", "--lr-decay-style", "constant", "--hidden-dropout", "0",
        "--attention-dropout", "0", "--seed", "1234", "--distributed-backend", "gloo", "--optimization-level", "0",
        "--use-cpu-initialization", "--weight-decay", "0.01", "--untie-embeddings-and-output-weights",
        "--use-distributed-optimizer", "--train-iters", "5"]


def _run(rank, world, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.training import pretrain
    hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                    args_list=ARGS + list(extra))
    return [h["lm loss"] for h in hist]


def test_swap_optimizer_is_exact():
    base = run_distributed(_run, 1, [])[0]
    swap = run_distributed(_run, 1, ["--swap-optimizer", "--swap-optimizer-times", "4"])[0]
    assert swap == pytest.approx(base, abs=1e-6)


def test_quantised_states_and_ema_and_muon_train():
    base = run_distributed(_run, 1, [])[0]
    q = run_distributed(_run, 1, ["--quant-states", "fp8"])[0]
    assert abs(q[-1] - base[-1]) < 0.05 and q[-1] < q[0] + 0.05
    mx = run_distributed(_run, 1, ["--quant-states", "mxfp8"])[0]
    assert abs(mx[-1] - base[-1]) < 0.05
    ema = run_distributed(_run, 1, ["--optimizer-selection", "fused_ema_adamw"])[0]
    assert ema == pytest.approx(base, abs=1e-6)            # EMA tracking does not change the trajectory
    mu = run_distributed(_run, 1, ["--optimizer", "muon", "--lr", "1e-3"])[0]
    assert all(x == x for x in mu)


def test_swap_muon_matches_muon():
    import torch
    from mindspeed_b200.optimizer.muon import Muon, SwapMuon
    torch.manual_seed(0)
    w1 = torch.nn.Parameter(torch.randn(16, 24))
    w2 = torch.nn.Parameter(w1.detach().clone())
    a, b = Muon([w1], lr=0.05, weight_decay=0.01), SwapMuon([w2], lr=0.05, weight_decay=0.01)
    for step in range(4):
        g = torch.randn(16, 24, generator=torch.Generator().manual_seed(step))
        w1.grad, w2.grad = g.clone(), g.clone()
        a.step(); b.step()
    assert torch.allclose(w1, w2, atol=1e-6)
    assert b.state[w2]["momentum_host"].device.type == "cpu" and "momentum_buffer" not in b.state[w2]
