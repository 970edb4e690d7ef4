"""A device-side bounded wait that expired leaves a code in the status word; the training loop must turn it into an
error instead of carrying on with outputs that were never computed.  The word is set on the host here."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402
from test_pipeline_cpu import BASE  # noqa: E402


def test_check_kernel_status_raises_once_and_clears():
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.training.training import check_kernel_status
    G._status["host-test"] = torch.tensor([0x21, 0, 0, 0], dtype=torch.int32)
    try:
        with pytest.raises(RuntimeError, match="0x21"):
            check_kernel_status()
        check_kernel_status()            # the word was cleared: the next check passes
    finally:
        G._status.pop("host-test", None)


def _train_with_status(rank, world):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train
    args = initialize_megatron(args_list=BASE + ["--train-iters", "3"])
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    it = pg.train_valid_test_datasets_provider(args)
    hist = train(pg.forward_step, model, opt, sched, it)            # healthy: runs to the end
    assert len(hist) == 3
    args.iteration = 0
    G._status["host-test"] = torch.tensor([0x140, 0, 0, 0], dtype=torch.int32)   # "peer 0x40 never arrived"
    try:
        train(pg.forward_step, model, opt, sched, it)
    except RuntimeError as e:
        return str(e)
    return "no error"


def test_train_raises_when_a_wait_timed_out():
    msg = run_distributed(_train_with_status, 1)[0]
    assert "0x140" in msg and "time-out" in msg, msg
