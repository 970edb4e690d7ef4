"""Quantisation-aware distillation through the training entry point: a frozen teacher read from a checkpoint, the student
trained on the KL divergence from its logits, the cross entropy reported only."""
import os
import sys
import tempfile

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402
from test_checkpoint_cpu import ARGS  # noqa: E402


def _run(rank, world, tp, iters, save, load, more=()):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.qat import qad
    from mindspeed_b200.training import pretrain
    qad.reset()
    extra = ["--tensor-model-parallel-size", str(tp), "--train-iters", str(iters)]
    extra += (["--save", save] if save else []) + (["--load", load] if load else []) + list(more)
    hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                    args_list=ARGS + extra)
    frozen = True
    if qad._TEACHER is not None:
        t = qad._TEACHER.teacher
        frozen = (not t.training) and all(not p.requires_grad and p.grad is None for p in t.parameters())
    return [h["lm loss"] for h in hist], [h.get("kl loss") for h in hist], frozen


def test_kl_from_logits_matches_torch_and_scales_with_temperature():
    from mindspeed_b200.qat.qad import kl_from_logits
    g = torch.Generator().manual_seed(0)
    s, t = torch.randn(2, 6, 50, generator=g, requires_grad=True), torch.randn(2, 6, 50, generator=g)
    mask = (torch.rand(2, 6, generator=g) > 0.3).float()
    for T in (1.0, 2.5):
        ref = torch.nn.functional.kl_div(torch.log_softmax(s / T, -1), torch.log_softmax(t / T, -1), reduction="none",
                                         log_target=True).sum(-1) * T * T
        got, n = kl_from_logits(s, t, mask, T, "mean")
        assert torch.allclose(got, (ref * mask).sum() / mask.sum(), atol=1e-6) and float(n) == float(mask.sum())
        got, _ = kl_from_logits(s, t, mask, T, "sum")
        assert torch.allclose(got, (ref * mask).sum(), atol=1e-5)
    assert float(kl_from_logits(s, s.detach(), None, 1.0, "mean")[0]) < 1e-7


def test_student_distils_from_a_checkpointed_teacher():
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_run, 1, 1, 2, d, None)                                    # the teacher: two steps, saved
        # student starts from the teacher's weights: zero divergence before the first update, none after updates by a zero loss
        lm, kl, frozen = run_distributed(_run, 1, 1, 2, None, d, ["--qad-enable", "--qad-teacher-load", d, "--finetune"])[0]
        assert frozen and kl[0] == pytest.approx(0.0, abs=1e-6) and all(v > 3.0 for v in lm)
        # fake-quantised student: a positive divergence from the first step on; after the first updates disturb the student
        # training pulls it back towards the teacher, which stays frozen and full precision
        q = ["--qad-enable", "--qad-teacher-load", d, "--finetune", "--qat-scheme", "w4a16", "--qat-quant-block-size", "32",
             "--lr", "2e-3"]
        lm, kl, frozen = run_distributed(_run, 1, 1, 8, None, d, q)[0]
        assert frozen and kl[0] > 1e-6 and kl[-1] < 0.5 * max(kl), kl
        # vocabulary-parallel logits over two ranks: the same loss
        lm2, kl2, frozen2 = run_distributed(_run, 2, 2, 2, None, d, q)[0]
        assert frozen2 and kl2[0] == pytest.approx(kl[0], rel=2e-3), (kl, kl2)
        # temperature and weight enter as T^2 and a plain factor
        _, klw, _ = run_distributed(_run, 1, 1, 1, None, d, q + ["--kl-loss-weight", "0.0"])[0]
        assert klw[0] == pytest.approx(kl[0], rel=1e-5)                            # the reported value is unweighted


def test_flags_validate(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "2")
    from mindspeed_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128"]
    validate_args(parse_args(args_list=base + ["--qad-enable", "--qad-teacher-load", "/x", "--kl-loss-reduction", "sum"]))
    a = validate_args(parse_args(args_list=base + ["--qad-enable", "--no-qad-enable"]))
    assert not a.qad_enable
    for extra, msg in ((["--qad-enable"], "qad-teacher-load"),
                       (["--qad-enable", "--qad-teacher-load", "/x", "--kl-temperature", "0"], "kl-temperature"),
                       (["--qad-enable", "--qad-teacher-load", "/x", "--kl-loss-weight", "-1"], "kl-loss-weight"),
                       (["--qad-enable", "--qad-teacher-load", "/x", "--num-experts", "4"], "dense"),
                       (["--qad-enable", "--qad-teacher-load", "/x", "--pipeline-model-parallel-size", "2"], "pipeline")):
        with pytest.raises(AssertionError, match=msg):
            validate_args(parse_args(args_list=base + extra))
