"""Training-loop extras wired to their flags: evaluation loop, scalar writer, learning-rate warm-up fraction, collective-free
fault dumps, per-layer recompute counts."""
import json
import os
import sys
import tempfile

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402
from test_pipeline_cpu import BASE  # noqa: E402


def _train_with(rank, world, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import io
    from contextlib import redirect_stdout
    import pretrain_gpt as pg
    from mindspeed_b200.training import pretrain
    buf = io.StringIO()
    with redirect_stdout(buf):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + list(extra))
    return [h["lm loss"] for h in hist], buf.getvalue()


def test_eval_loop_and_scalar_file():
    with tempfile.TemporaryDirectory() as d:
        losses, out = run_distributed(_train_with, 1, ["--train-iters", "4", "--eval-interval", "2", "--eval-iters", "2",
                                                       "--tensorboard-dir", d, "--log-interval", "1"])[0]
        assert out.count("validation at iteration") == 2
        rows = [json.loads(l) for l in open(os.path.join(d, "scalars.jsonl"))]
        tags = {r["tag"] for r in rows}
        assert {"lm loss", "learning-rate", "lm loss validation"} <= tags
        assert max(r["step"] for r in rows) == 4


def test_scalar_sinks_follow_the_logging_flags():
    with tempfile.TemporaryDirectory() as d:
        _, out = run_distributed(_train_with, 1, ["--train-iters", "4", "--eval-interval", "4", "--eval-iters", "1", "--tensorboard-dir", d,
                                                  "--tensorboard-log-interval", "2", "--log-world-size-to-tensorboard",
                                                  "--log-validation-ppl-to-tensorboard", "--log-timers-to-tensorboard",
                                                  "--no-log-learning-rate-to-tensorboard", "--wandb-project", "unit-test"])[0]
        rows = [json.loads(l) for l in open(os.path.join(d, "scalars.jsonl"))]
        tags = {r["tag"] for r in rows}
        assert {"world-size", "lm loss", "tokens-per-second", "lm loss validation ppl"} <= tags and "learning-rate" not in tags
        assert sorted({r["step"] for r in rows if r["tag"] == "lm loss"}) == [2, 4]          # every second iteration
        ppl = next(r["value"] for r in rows if r["tag"] == "lm loss validation ppl")
        val = next(r["value"] for r in rows if r["tag"] == "lm loss validation")
        assert ppl == pytest.approx(__import__("math").exp(val), rel=1e-6)
        try:
            import wandb  # noqa: F401
        except ImportError:
            assert "wandb package is not usable" in out


def test_lr_warmup_fraction_sets_warmup_steps():
    from mindspeed_b200.training.training import OptimizerParamScheduler

    class Opt:
        param_groups = [{"lr": 0.0}]
    s = OptimizerParamScheduler(Opt(), 1.0, 0.0, int(0.25 * 8), 8, "linear")
    lrs = []
    for _ in range(3):
        s.step(1)
        lrs.append(Opt.param_groups[0]["lr"])
    assert lrs[0] == pytest.approx(0.5) and lrs[1] == pytest.approx(1.0) and lrs[2] < 1.0
    losses_a, _ = run_distributed(_train_with, 1, ["--train-iters", "3", "--lr-warmup-fraction", "0.5", "--lr-decay-iters", "4"])[0]
    losses_b, _ = run_distributed(_train_with, 1, ["--train-iters", "3", "--lr-warmup-iters", "2", "--lr-decay-iters", "4"])[0]
    assert losses_a == pytest.approx(losses_b, abs=1e-7)


def _dump_roundtrip(rank, world, d):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.checkpointing import load_fault_dump, save_fault_dump, wait_for_fault_dump
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    args = initialize_megatron(args_list=BASE + ["--tensor-model-parallel-size", str(world), "--train-iters", "4"])
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    it = pg.train_valid_test_datasets_provider(args)
    for _ in range(2):
        train_step(pg.forward_step, it, model, opt, sched)
    # each rank dumps on its own (no collective), twice, keeping one
    save_fault_dump(1, model, opt, d, keep=1)
    save_fault_dump(2, model, opt, d, keep=1)
    before = {n: p.detach().clone() for n, p in model[0].module.named_parameters()}
    m_before = [st.m.clone() for st in opt._all_states()]
    for p in model[0].module.parameters():
        p.data.zero_()
    for st in opt._all_states():
        st.m.zero_()
    found = wait_for_fault_dump(d, [rank], timeout_s=5)
    assert found is not None and found.endswith("iter_0000002")
    assert load_fault_dump(model, opt, found) == 2
    ok = all(torch.equal(before[n], p.detach()) for n, p in model[0].module.named_parameters())
    ok = ok and all(torch.equal(a, st.m) for a, st in zip(m_before, opt._all_states()))
    kept = sorted(x for x in os.listdir(d) if os.path.isdir(os.path.join(d, x, f"rank_{rank}")))
    return ok, kept


def test_fault_dump_is_collective_free_and_restores_state():
    with tempfile.TemporaryDirectory() as d:
        res = run_distributed(_dump_roundtrip, 2, d)
        assert all(r[0] for r in res), res
        assert all(r[1] == ["iter_0000002"] for r in res), res
