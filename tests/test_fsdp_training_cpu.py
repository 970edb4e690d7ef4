"""--layerzero / --fsdp2-config-path in the training loop: two gloo data-parallel ranks follow the bucketed-DDP run."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402
from test_pipeline_cpu import BASE  # noqa: E402


def _train(rank, world, extra):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import SyntheticGPTDataset
    args = initialize_megatron(args_list=[a for a in BASE if a != "--no-gradient-accumulation-fusion"] + ["--clip-grad", "1.0"] + list(extra))
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
    dp_r, dp_n = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
    nmb = args.global_batch_size // (args.micro_batch_size * dp_n)
    state = {"i": 0}

    class It:
        def __iter__(self):
            return self

        def __next__(self):
            # global micro-batch index -> the same samples whatever the data-parallel wrapper is
            step, k = divmod(state["i"], nmb)
            state["i"] += 1
            item = ds[step * nmb * dp_n + k * dp_n + dp_r]
            return {kk: v.unsqueeze(0) for kk, v in item.items()}

    out = []
    for _ in range(3):
        ld, *_ = train_step(pg.forward_step, It(), model, opt, sched)
        out.append(float(ld["lm loss"]))
    return out, type(model[0]).__name__


@pytest.mark.parametrize("extra", [["--layerzero"], ["--fsdp2-config-path", "PLAN"]])
def test_fsdp_flags_follow_ddp(extra, tmp_path):
    if "PLAN" in extra:
        plan = tmp_path / "plan.yaml"
        plan.write_text("fsdp:\n  wrap: [TransformerLayer]\n  reshard_after_forward: true\n")
        extra = ["--fsdp2-config-path", str(plan)]
    ref = run_distributed(_train, 2, [])
    got = run_distributed(_train, 2, extra)
    assert ref[0][1] == "DistributedDataParallel" and got[0][1] == "FullyShardedDataParallel"
    for r in range(2):
        for a, b in zip(ref[r][0], got[r][0]):
            assert abs(a - b) < 5e-4 * max(1.0, abs(a)), (ref, got)
