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
        out.append(float(ld["lm loss"]) if "lm loss" in ld else None)     # only the last pipeline stage sees the loss
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


@pytest.mark.parametrize("layout", [
    ["--tensor-model-parallel-size", "2", "--sequence-parallel"],           # FSDP over the 2 data-parallel ranks of each TP rank
    ["--pipeline-model-parallel-size", "2"],                                # FSDP-wrapped pipeline stages
])
def test_fsdp_with_tensor_and_pipeline_parallel_follows_ddp(layout):
    """--layerzero on 4 ranks with tensor (+ sequence) parallelism or pipeline stages: same losses and the same clipped
    gradient norm as bucketed DDP in the same layout (norm weights summed over the sequence slices, parameters duplicated
    over the tensor-parallel ranks counted once)."""
    ref = run_distributed(_train, 4, layout)
    got = run_distributed(_train, 4, layout + ["--layerzero"])
    assert got[0][1] == "FullyShardedDataParallel"
    ref_l = [r[0] for r in ref if r[0][0] is not None]
    got_l = [r[0] for r in got if r[0][0] is not None]
    for a, b in zip(ref_l[-1], got_l[-1]):
        assert abs(a - b) < 1e-3 * max(1.0, abs(a)), (ref_l, got_l)


def _fsdp_ckpt(rank, world, d, phase, shard_size):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch
    import pretrain_gpt as pg
    from mindspeed_b200.checkpointing import load_checkpoint, save_checkpoint
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import SyntheticGPTDataset
    plan = os.path.join(d, f"plan{shard_size}.yaml")
    if rank == 0:
        with open(plan, "w") as f:
            f.write(f"fsdp:\n  wrap: [TransformerLayer]\n  shard_size: {shard_size}\n  zero1_over_replicas: {'true' if shard_size < world else 'false'}\n")
    args = initialize_megatron(args_list=[a for a in BASE if a != "--no-gradient-accumulation-fusion"] +
                               ["--clip-grad", "1.0", "--fsdp2-config-path", plan, "--save", d, "--load", d])
    torch.distributed.barrier()
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)

    class It:
        i = 0

        def __iter__(self):
            return self

        def __next__(self):
            It.i += 1
            return {k: v.unsqueeze(0) for k, v in ds[It.i * world + rank].items()}

    if phase == "save":
        for _ in range(2):
            train_step(pg.forward_step, It(), model, opt, sched)
        save_checkpoint(2, model, opt, sched, args)
        It.i = 100
        ld, *_ = train_step(pg.forward_step, It(), model, opt, sched)
        return float(ld["lm loss"]), model[0].full_state_dict()["decoder.layers.0.mlp.linear_fc1.weight"].sum().item()
    it = load_checkpoint(model, opt, sched, args=args)
    assert it == 2
    It.i = 100
    ld, *_ = train_step(pg.forward_step, It(), model, opt, sched)
    return float(ld["lm loss"]), model[0].full_state_dict()["decoder.layers.0.mlp.linear_fc1.weight"].sum().item()


def test_fsdp_sharded_checkpoint_reloads_under_another_shard_size(tmp_path):
    """Parameters and Adam moments saved from 4-way sharding are read back into 2-way sharding x 2 replicas with the
    optimizer state also split over the replicas (LayerZeRO layout): the next step is the same."""
    d = str(tmp_path)
    saved = run_distributed(_fsdp_ckpt, 4, d, "save", 4)
    loaded = run_distributed(_fsdp_ckpt, 4, d, "load", 2)
    for (l0, w0), (l1, w1) in zip(saved, loaded):
        assert abs(l0 - l1) < 1e-5 * max(1.0, abs(l0)), (saved, loaded)
        assert abs(w0 - w1) < 1e-4 * max(1.0, abs(w0)), (saved, loaded)


def _probe(rank, world, extra, save_dir, steps):
    """Train ``steps`` steps (optionally save), then report the loss of one more step on fixed samples."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.checkpointing import save_checkpoint
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import SyntheticGPTDataset
    base = [a for a in BASE if a != "--no-gradient-accumulation-fusion"]
    base[base.index("--global-batch-size") + 1] = "4"
    base[base.index("--num-layers") + 1] = "2"
    args = initialize_megatron(args_list=base + ["--clip-grad", "1.0"] + list(extra))
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
    dp_r, dp_n = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()

    class It:
        base, m = 0, 0

        def __iter__(self):
            return self

        def __next__(self):
            i = It.base + It.m * dp_n + dp_r                      # the same global samples for every parallel layout
            It.m += 1
            return {k: v.unsqueeze(0) for k, v in ds[i].items()}

    for s in range(steps):
        It.base, It.m = 4 * s, 0
        train_step(pg.forward_step, It(), model, opt, sched)
    if save_dir and steps:
        save_checkpoint(steps, model, opt, sched, args, save_dir=save_dir)
    It.base, It.m = 1000, 0
    ld, *_ = train_step(pg.forward_step, It(), model, opt, sched)
    return float(ld["lm loss"])


@pytest.mark.parametrize("world,tp", [(2, 1), (4, 2)])
def test_fully_sharded_checkpoint_converts_to_the_regular_layout(tmp_path, world, tp):
    """A LayerZeRO checkpoint (flat per-parameter shards; with tensor parallelism one set per tensor-parallel rank) is
    converted offline and read by a plain single-rank model: the loss on fixed samples is the sharded run's."""
    import torch
    from mindspeed_b200.checkpointing import convert_fsdp
    src, dst = str(tmp_path / "fsdp"), str(tmp_path / "plain")
    flags = ["--layerzero", "--lr", "1e-2"] + (["--tensor-model-parallel-size", str(tp), "--sequence-parallel"] if tp > 1 else [])
    sharded = run_distributed(_probe, world, flags, src, 2)[0]
    assert convert_fsdp.main(["--input_folder", src, "--output_folder", dst, "--target_tp", "1", "--target_pp", "1"]) == 0
    common = torch.load(os.path.join(dst, "iter_0000002", "common.pt"), weights_only=False)
    assert common["args"]["tensor_model_parallel_size"] == 1 and "fsdp_layout" not in common
    assert common["converted_from"]["source_tp"] == tp
    plain = run_distributed(_probe, 1, ["--load", dst, "--finetune"], None, 0)[0]
    assert abs(plain - sharded) < 2e-5 * max(1.0, abs(sharded)), (sharded, plain)
    untrained = run_distributed(_probe, 1, [], None, 0)[0]
    assert abs(untrained - sharded) > 1e-3                        # the probe does depend on the trained weights


def test_gated_projection_rows_regroup_between_tensor_parallel_sizes():
    import torch
    from mindspeed_b200.checkpointing.convert_fsdp import regroup_gated
    gate, up = torch.arange(8.0).view(8, 1), 100 + torch.arange(8.0).view(8, 1)
    per_rank = lambda tp: torch.cat([torch.cat((g, u)) for g, u in zip(gate.chunk(tp), up.chunk(tp))])
    for a in (1, 2, 4):
        for b in (1, 2, 4):
            assert torch.equal(regroup_gated(per_rank(a), a, b), per_rank(b)), (a, b)
    w = torch.randn(3, 8)
    assert torch.equal(regroup_gated(regroup_gated(w, 2, 4, dim=1), 4, 2, dim=1), w)
