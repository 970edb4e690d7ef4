"""Tiny GPT on CPU/gloo: world 2, TP=2, fp32, 10 Adam steps; loss curve must match the unsharded run.

Shape: 2 layers, hidden 256, 4 heads, FFN 1024 GeLU, LayerNorm, learned positions, vocab 1024, seq 128,
micro-batch 2, global batch 4, ids uniform in [0,1024) from seed 1234, N(0,0.02) init, lr 1e-4.
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

ARGS = ["--num-layers", "2", "--hidden-size", "256", "--num-attention-heads", "4", "--ffn-hidden-size", "1024",
        "--seq-length", "128", "--max-position-embeddings", "128", "--micro-batch-size", "2", "--global-batch-size", "4",
        "--vocab-size", "1024", "--make-vocab-size-divisible-by", "1", "--train-iters", "10", "--lr", "1e-4",
        "--lr-decay-style", "constant", "--hidden-dropout", "0", "--attention-dropout", "0", "--seed", "1234",
        "--init-method-std", "0.02", "--distributed-backend", "gloo", "--optimization-level", "0", "--use-cpu-initialization",
        "--weight-decay", "0.0", "--clip-grad", "1.0", "--untie-embeddings-and-output-weights"]


def _train(rank, world, tp, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.training import pretrain
    hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                    args_list=ARGS + ["--tensor-model-parallel-size", str(tp)] + list(extra))
    return [h["lm loss"] for h in hist]


def test_tp2_matches_unsharded():
    ref = run_distributed(_train, 1, 1, [])[0]
    tp2 = run_distributed(_train, 2, 2, [])
    assert len(ref) == 10
    assert ref[-1] < ref[0], "loss must go down"
    for a, b in zip(ref, tp2[0]):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (ref, tp2[0])
    assert tp2[0] == pytest.approx(tp2[1], abs=1e-7)


def test_tp2_sequence_parallel_matches():
    ref = run_distributed(_train, 1, 1, [])[0]
    sp = run_distributed(_train, 2, 2, ["--sequence-parallel"])[0]
    for a, b in zip(ref, sp):
        assert abs(a - b) <= 2e-5 * max(1.0, abs(a)), (ref, sp)
