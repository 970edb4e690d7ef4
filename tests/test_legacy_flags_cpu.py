"""Older spellings and small legacy options: each is rewritten onto, or implemented next to, the feature it names."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASE = ["--num-layers", "4", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
        "--micro-batch-size", "1", "--vocab-size", "128"]


def _args(extra, world=1, monkeypatch=None):
    from mindspeed_b200.training.arguments import parse_args, validate_args
    if monkeypatch is not None:
        monkeypatch.setenv("WORLD_SIZE", str(world))
    return validate_args(parse_args(args_list=BASE + list(extra)))


def test_older_spellings_are_rewritten(monkeypatch, tmp_path):
    a = _args(["--tensor-model-parallel-size", "4", "--use-nd-matmul", "--nd1-dim1-size", "2", "--nd2-dim1-size", "2"], 4, monkeypatch)
    assert a.tp_2d and (a.tp_x, a.tp_y) == (2, 2)
    with pytest.raises(AssertionError, match="must equal"):
        _args(["--tensor-model-parallel-size", "4", "--use-nd-matmul", "--nd1-dim1-size", "2", "--nd2-dim1-size", "1"], 4, monkeypatch)
    a = _args(["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--optimize-vpp-send-recv-comm"],
              2, monkeypatch)
    assert a.optimize_send_recv_comm
    a = _args(["--enable-zero3"], 2, monkeypatch)
    assert a.layerzero
    a = _args(["--multi-head-latent-attention", "--rope-scaling-type", "yarn", "--yarn-scaling-factor", "8"], 1, monkeypatch)
    assert a.rope_scaling_factor == 8
    a = _args(["--num-experts", "4", "--moe-model-type", "deepspeed_moe", "--expert-interval", "2"], 1, monkeypatch)
    assert a.moe_layer_freq == [0, 1, 0, 1]
    with pytest.raises(AssertionError, match="deepspeed_moe"):
        _args(["--num-experts", "4", "--expert-interval", "2"], 1, monkeypatch)
    cfgf = tmp_path / "more.json"
    cfgf.write_text(json.dumps({"--add-dense-bias": True, "kl_temperature": 2.5}))
    a = _args(["--additional-config", str(cfgf)], 1, monkeypatch)
    assert a.add_dense_bias is True and a.kl_temperature == 2.5
    cfgf.write_text("no_such_argument: 1\n")
    with pytest.raises(AssertionError, match="unknown argument"):
        _args(["--additional-config", str(cfgf)], 1, monkeypatch)
    a = _args(["--optimized-mbs-list", "[2,1,1]"], 1, monkeypatch)
    assert a.micro_batch_sizes == [2, 1, 1] and a.global_batch_size == 4 and a.micro_batch_size == 2
    with pytest.raises(AssertionError, match="deepspeed_moe"):
        _args(["--ampipe-degree", "2"], 1, monkeypatch)
    with pytest.raises(AssertionError, match="use-nanopipe"):
        _args(["--use-nanopipe"], 1, monkeypatch)


def test_random_token_selection_keeps_capacity_and_is_not_position_biased():
    from mindspeed_b200.legacy_moe.gate import top1gating
    torch.manual_seed(0)
    S, E = 64, 2
    logits = torch.zeros(S, E)
    logits[:, 0] = 1.0                                             # every token wants expert 0: capacity 32 * cf
    _, comb, mask, counts = top1gating(logits, capacity_factor=0.5, min_capacity=4)
    kept = mask.any(-1)[:, 0].nonzero().flatten()
    assert kept.tolist() == list(range(16))                        # sequence order: the first 16
    picks = []
    for _ in range(4):
        _, comb, mask, _ = top1gating(logits, capacity_factor=0.5, min_capacity=4, use_rts=True)
        m = mask[:, 0]                                             # [S, C]
        assert int(m.any(-1).sum()) == 16 and int(m.sum(0).max()) == 1          # 16 kept, one token per capacity slot
        picks.append(tuple(m.any(-1).nonzero().flatten().tolist()))
    assert len(set(picks)) > 1 and any(max(p) >= 32 for p in picks)
    # under capacity nothing is dropped either way
    lg = torch.randn(16, 4)
    a = top1gating(lg, capacity_factor=4.0)[1]
    b = top1gating(lg, capacity_factor=4.0, use_rts=True)[1]
    assert torch.equal(a.sum(-1), b.sum(-1))


def _train_moe(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE as TB
    from mindspeed_b200.parallel.moe.moe_layer import MoELayer
    from mindspeed_b200.training import pretrain
    layers = []
    orig = MoELayer.__init__

    def spy(self, *a, **kw):
        orig(self, *a, **kw)
        layers.append(self)
    MoELayer.__init__ = spy
    flags = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-token-dispatcher-type", "alltoall", "--moe-grouped-gemm",
             "--moe-aux-loss-coeff", "0.01", "--train-iters", "4"]
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=TB + flags + list(extra))
    MoELayer.__init__ = orig
    return [h.get("lm loss") for h in hist], [l.recomputed_steps for l in layers], [{k: float(v) for k, v in h.items() if "balancing" in k} for h in hist]


def test_moe_recompute_only_on_unbalanced_steps_changes_no_numbers():
    from dist_utils import run_distributed
    plain, r0, aux = run_distributed(_train_moe, 1, [])[0]
    # the routers' load-balancing loss is reported per log line: mean over the MoE layers, >= 1 x coefficient when unbalanced
    assert all(set(a) == {"load_balancing_loss"} and 0.0099 < a["load_balancing_loss"] < 0.05 for a in aux), aux
    assert set(r0) == {0}
    # an unreachable threshold: only the very first forward of every layer (no history yet) recomputes
    hi, r1, _ = run_distributed(_train_moe, 1, ["--moe-adaptive-recompute-activation", "--moe-adaptive-recompute-activation-scale", "100"])[0]
    assert set(r1) == {1} and hi == pytest.approx(plain, abs=1e-6)
    # a threshold every step exceeds: every forward (4 steps x 8 micro-batches) recomputes
    lo, r2, _ = run_distributed(_train_moe, 1, ["--moe-adaptive-recompute-activation", "--moe-adaptive-recompute-activation-scale", "0.01"])[0]
    assert set(r2) == {32} and lo == pytest.approx(plain, abs=1e-6)
    # two pipeline stages: every stage joins the reduction, every layer is reported once
    pp, _, aux_pp = run_distributed(_train_moe, 2, ["--pipeline-model-parallel-size", "2", "--moe-per-layer-logging"])[1]
    # (the two stages draw their initial weights independently, so the values differ from the one-stage run)
    assert all(0.0099 < a["load_balancing_loss"] < 0.05 for a in aux_pp), aux_pp
    per_layer = [aux_pp[0][f"load_balancing_loss layer {i}"] for i in (1, 2, 3, 4)]
    assert abs(sum(per_layer) / 4 - aux_pp[0]["load_balancing_loss"]) < 1e-6 and all(x > 0.0099 for x in per_layer)


def test_dense_bias_flag_adds_the_projection_bias():
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.models.attention import SelfAttention
    from mindspeed_b200.parallel import parallel_state as ps
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", str(__import__("dist_utils")._free_port()))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1, 1)
    kw = dict(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True, optimization_level=0, add_bias_linear=False)
    cfg = TransformerConfig(**kw)
    assert SelfAttention(cfg).linear_proj.bias is None
    cfg2 = TransformerConfig(**kw)
    cfg2.add_dense_bias = True
    assert SelfAttention(cfg2).linear_proj.bias is not None and SelfAttention(cfg2).linear_qkv.bias is None
    ps.destroy_model_parallel()


def _train_mbs(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE as TB, _canonical_init
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    args = initialize_megatron(args_list=list(TB) + list(extra))
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    _canonical_init(model)
    if hasattr(opt, "reload_model_params"):
        opt.reload_model_params()
    it = pg.train_valid_test_datasets_provider(args)
    out = []
    with redirect_stdout(io.StringIO()):
        for _ in range(2):
            ld, *_ = train_step(pg.forward_step, [it] * len(model) if len(model) > 1 else it, model, opt, sched)
            out.append(float(ld["lm loss"]) if "lm loss" in ld else None)
    from mindspeed_b200.parallel.pipeline import schedules as S
    if S._STORED_PLANS:
        out.append("stored plan")
    return out


def test_micro_batches_of_different_sizes_give_the_same_step():
    """--optimized-mbs-list: 8 samples per step as micro-batches of 3 + 1 + 2 + 2 equal eight micro-batches of one sample,
    without pipeline parallelism and across two stages (messages sized per micro-batch)."""
    from dist_utils import run_distributed
    ref = run_distributed(_train_mbs, 1, [])[0]
    got = run_distributed(_train_mbs, 1, ["--optimized-mbs-list", "[3,1,2,2]"])[0]
    assert got == pytest.approx(ref, abs=2e-5), (ref, got)
    pp = run_distributed(_train_mbs, 2, ["--pipeline-model-parallel-size", "2", "--optimized-mbs-list", "3,1,2,2"])
    have = [r for r in pp if r[0] is not None][0]
    assert have == pytest.approx(ref, abs=2e-4), (ref, have)
    from mindspeed_b200.training.arguments import parse_args, validate_args
    with pytest.raises(AssertionError, match="sums to"):
        validate_args(parse_args(args_list=BASE + ["--global-batch-size", "8", "--optimized-mbs-list", "[3,1]"]))


def test_stored_pipeline_schedule_runs_as_given():
    """--pp-schedule-list: an all-forward-then-all-backward order (not the 1F1B default) gives the same step; an order in
    which the two ranks wait for each other is refused at start-up."""
    import json
    from dist_utils import run_distributed
    from mindspeed_b200.parallel.pipeline.plan import plan_from_stage_lists
    n = 8
    gpipe = {f"stage{r}": [f"F{i}" for i in range(1, n + 1)] + [f"B{i}" for i in range(1, n + 1)] for r in range(2)}
    plan = plan_from_stage_lists(2, n, gpipe)
    assert [o.kind for slot in plan.table[1] for o in slot][:n] == ["F"] * n
    ref = run_distributed(_train_mbs, 1, [])[0]
    got = [r for r in run_distributed(_train_mbs, 2, ["--pipeline-model-parallel-size", "2", "--pp-schedule-list", json.dumps(gpipe)])
           if r[0] is not None][0]
    assert got[-1] == "stored plan" and got[:-1] == pytest.approx(ref, abs=2e-4), (ref, got)
    bad = {"stage0": ["F1", "B1"] + [t for i in range(2, n + 1) for t in (f"F{i}", f"B{i}")],
           "stage1": [f"F{i}" for i in range(n, 0, -1)] + [f"B{i}" for i in range(1, n + 1)]}
    with pytest.raises(RuntimeError, match="deadlocks"):
        plan_from_stage_lists(2, n, bad)
    with pytest.raises(ValueError, match="expected"):
        plan_from_stage_lists(2, n, {"stage0": ["F1", "B1"], "stage1": ["F1", "B1"]})
    with pytest.raises(ValueError, match="before its forward"):
        plan_from_stage_lists(2, 1, {"stage0": ["B1", "F1"], "stage1": ["F1", "B1"]})

