"""Checkpoint save / resume / reshard on CPU/gloo."""
import os
import sys
import tempfile

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

ARGS = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--ffn-hidden-size", "128", "--seq-length", "32",
        "--max-position-embeddings", "32", "--micro-batch-size", "2", "--global-batch-size", "4", "--vocab-size", "128",
        "--make-vocab-size-divisible-by", "1", "--lr", "1e-3", "--lr-decay-style", "constant", "--hidden-dropout", "0",
        "--attention-dropout", "0", "--seed", "1234", "--distributed-backend", "gloo", "--optimization-level", "0",
        "--use-cpu-initialization", "--weight-decay", "0.01", "--untie-embeddings-and-output-weights", "--use-distributed-optimizer"]


def _run(rank, world, tp, iters, save, load, more=()):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.training import pretrain
    extra = ["--tensor-model-parallel-size", str(tp), "--train-iters", str(iters)]
    if save:
        extra += ["--save", save]
    if load:
        extra += ["--load", load]
    extra += list(more)
    hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                    args_list=ARGS + extra)
    return [h["lm loss"] for h in hist]


def test_resume_matches_uninterrupted_run():
    with tempfile.TemporaryDirectory() as d:
        full = run_distributed(_run, 2, 2, 4, None, None)[0]
        first = run_distributed(_run, 2, 2, 2, d, None)[0]
        assert os.path.exists(os.path.join(d, "latest_checkpointed_iteration.txt"))
        assert os.path.exists(os.path.join(d, "iter_0000002", ".metadata"))
        assert os.path.exists(os.path.join(d, "iter_0000002", "common.pt"))
        second = run_distributed(_run, 2, 2, 4, None, d)[0]
        assert first == pytest.approx(full[:2], abs=1e-6)
        assert second == pytest.approx(full[2:], abs=1e-5)


def test_reshard_tp2_to_tp1_and_dp2():
    """Saved under TP=2, loaded under TP=1 x DP=2: same model, same optimizer state -> same continued losses."""
    with tempfile.TemporaryDirectory() as d:
        full = run_distributed(_run, 2, 2, 4, None, None)[0]
        run_distributed(_run, 2, 2, 2, d, None)
        # model weights reshard across TP; optimizer state needs the same TP, so continue without it on TP=1
        cont = run_distributed(_run, 2, 1, 3, None, d, ["--no-load-optim"])
        assert len(cont[0]) == 1
        # the first continued step's loss is computed with exactly the saved weights
        assert cont[0][0] == pytest.approx(full[2], abs=2e-4)


def test_files_are_torch_distributed_checkpoint_with_megatron_style_keys():
    """The directory is readable by plain torch.distributed.checkpoint, keys carry no chunk prefix and per-layer tensors
    are stacked along a leading layer axis; ``--async-save`` writes the same files from a background thread."""
    from torch.distributed.checkpoint import FileSystemReader
    for more in ([], ["--async-save"]):
        with tempfile.TemporaryDirectory() as d:
            run_distributed(_run, 2, 2, 2, d, None, more)
            path = os.path.join(d, "iter_0000002")
            assert sorted(f for f in os.listdir(path) if f.endswith(".distcp")) == ["__0_0.distcp", "__1_0.distcp"]
            md = FileSystemReader(path).read_metadata().state_dict_metadata
            qkv = md["decoder.layers.self_attention.linear_qkv.weight"]
            assert tuple(qkv.size) == (2, 3 * 64, 64) and len(qkv.chunks) == 4          # 2 layers x 2 tensor-parallel shards
            assert tuple(md["embedding.word_embeddings.weight"].size) == (128, 64)
            assert tuple(md["decoder.final_layernorm.weight"].size) == (64,)
            assert "optimizer.state.exp_avg.decoder.layers.mlp.linear_fc1.weight" in md
            assert not any(k.startswith("model.") for k in md)
            # a plain DCP load of one tensor, no framework code involved
            import torch.distributed.checkpoint as dcp
            t = {"decoder.final_layernorm.weight": torch.zeros(64)}
            dcp.load(t, storage_reader=FileSystemReader(path), no_dist=True)
            assert float(t["decoder.final_layernorm.weight"].abs().sum()) > 0


def test_async_save_resume_matches_uninterrupted_run():
    with tempfile.TemporaryDirectory() as d:
        full = run_distributed(_run, 2, 2, 4, None, None)[0]
        run_distributed(_run, 2, 2, 2, d, None, ["--async-save"])
        second = run_distributed(_run, 2, 2, 4, None, d)[0]
        assert second == pytest.approx(full[2:], abs=1e-5)


def _load_foreign(rank, world, tp, load):
    """Build the model under ``tp`` ranks, read a checkpoint some other writer produced, return the loss of one step."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.training import pretrain
    extra = ["--tensor-model-parallel-size", str(tp), "--train-iters", "1", "--load", load, "--finetune", "--lr", "0.0"]
    hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                    args_list=ARGS + extra)
    return hist[0]["lm loss"]


def test_checkpoint_written_by_plain_torch_dcp_with_megatron_key_names_loads():
    """A directory produced by nothing but ``torch.distributed.checkpoint.save`` over a {Megatron key: full tensor} dict -
    what a Megatron-core ``torch_dist`` writer stores for a model without tensor parallelism - is read under tensor
    parallelism 1 and 2: the loss equals the one of the model whose weights were written."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader, FileSystemWriter
    with tempfile.TemporaryDirectory() as own, tempfile.TemporaryDirectory() as foreign:
        run_distributed(_run, 1, 1, 2, own, None)                               # train two steps, save in this framework
        src = os.path.join(own, "iter_0000002")
        md = FileSystemReader(src).read_metadata().state_dict_metadata
        weights = {k: torch.empty(tuple(v.size), dtype=v.properties.dtype) for k, v in md.items()
                   if not k.startswith("optimizer.") and hasattr(v, "size")}
        dcp.load(weights, storage_reader=FileSystemReader(src), no_dist=True)   # full tensors under Megatron names
        assert "decoder.layers.mlp.linear_fc1.weight" in weights and weights["decoder.layers.mlp.linear_fc1.weight"].dim() == 3
        dst = os.path.join(foreign, "iter_0000007")
        os.makedirs(dst)
        dcp.save(weights, storage_writer=FileSystemWriter(dst), no_dist=True)   # the foreign writer: stock DCP only
        with open(os.path.join(foreign, "latest_checkpointed_iteration.txt"), "w") as f:
            f.write("7")
        ref = run_distributed(_load_foreign, 1, 1, own)[0]
        for tp in (1, 2):
            got = run_distributed(_load_foreign, tp, tp, foreign)[0]
            assert got == pytest.approx(ref, abs=2e-5), (tp, ref, got)
        assert ref != pytest.approx(run_distributed(_run, 1, 1, 1, None, None)[0][0], abs=1e-4)   # not the initial weights
