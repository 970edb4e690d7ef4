"""auto_settings beyond the analytic model: profile parsing, operator database, fitted communication lines, pruning."""
import os
import tempfile

import pytest


def _trace():
    ev = []
    t = 0.0

    def k(name, dur, tid=7, at=None):
        nonlocal t
        ts = t if at is None else at
        ev.append({"ph": "X", "cat": "kernel", "name": name, "ts": ts, "dur": dur, "tid": tid})
        if at is None:
            t += dur
    for _ in range(4):
        k("void gemm2_sm100_kernel<256,4,0,0,1>", 200.0)
        k("flash_fwd2_sm100_kernel", 100.0)
        start = t
        k("rmsnorm_fwd_kernel<bf16>", 50.0)
        # an all-to-all on another stream: half of it under the norm kernel, half exposed
        k("moe_dispatch_kernel", 100.0, tid=9, at=start)
        t = start + 100.0
    k("ncclDevKernel_AllReduce_Sum_f32", 80.0, tid=11)
    ev.append({"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5})
    return ev


def test_profile_parse_classes_and_exposed_time():
    from mindspeed_b200.auto_settings.profiling_parse import classify, summarize
    assert classify("void gemm2_comm_kernel<0,1>") == "tp_fused"
    assert classify("ncclDevKernel_ReduceScatter_Sum_bf16") == "dp_reduce"
    assert classify("nvjet_tst_128x256") == "gemm"
    s = summarize(_trace())
    assert s.ops["gemm"].calls == 4 and s.ops["gemm"].total_us == pytest.approx(800.0)
    assert s.ops["attention"].total_us == pytest.approx(400.0)
    a2a = s.ops["ep_a2a"]
    assert a2a.total_us == pytest.approx(400.0) and a2a.exposed_us == pytest.approx(200.0)     # 50 of each 100 us hidden
    assert s.ops["allreduce"].exposed_us == pytest.approx(80.0)
    assert "cpu_op" not in s.ops and "class" in s.table()


def test_operator_db_exact_scaled_and_persistent():
    from mindspeed_b200.auto_settings.operator_db import OperatorDB
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ops.sqlite")
        db = OperatorDB(path)
        db.record("gemm", (8192, 4096, 4096), 0.20, flops=2 * 8192 * 4096 * 4096)
        db.record("gemm", (8192, 4096, 4096), 0.22, flops=2 * 8192 * 4096 * 4096)
        assert db.exact("gemm", (8192, 4096, 4096)).ms == pytest.approx(0.21) and len(db) == 1
        # unseen shape: nearest entry scaled by FLOPs
        assert db.lookup("gemm", (8192, 8192, 4096), flops=2 * 8192 * 8192 * 4096) == pytest.approx(0.42)
        assert db.lookup("attention", (1, 1), flops=1e9) is None
        eff = db.efficiency("gemm", 1.4e15)
        assert 0.9 < eff < 1.0
        assert len(OperatorDB(path)) == 1                       # survives a restart


def test_comm_lines_fit_and_change_the_ranking():
    from mindspeed_b200.auto_settings.comm_predictors import CommPredictors, LinearModel
    from mindspeed_b200.auto_settings.hardware import Hardware
    from mindspeed_b200.auto_settings.operator_db import OperatorDB
    from mindspeed_b200.auto_settings.search_space import ModelDesc
    from mindspeed_b200.auto_settings.searcher import white_search
    lm = LinearModel()
    for x in (1e-4, 2e-4, 4e-4):
        lm.add(x, 2.0 * x + 3e-5)
    lm.fit()
    assert lm.w == pytest.approx(2.0, rel=1e-6) and lm.b == pytest.approx(3e-5, rel=1e-6)
    hw = Hardware()
    model = ModelDesc(32, 4096, 14336, 32, 8, 128256, 8192, 64)
    base = white_search(model, 8, hw, topk=3)
    assert base and all(e.fits for e in base)
    # measurements say: the fused tensor-parallel kernels hide nothing and run at a fifth of the link speed
    comm = CommPredictors(hw)
    for nbytes in (2e7, 5e7, 1e8):
        x = comm.x("mc2", nbytes, 8)
        comm.add_sample("mc2", nbytes, 8, 5.0 * x + 2e-5, 5.0 * x + 2e-5)
    comm.fit()
    db = OperatorDB()
    db.record("gemm", (8192, 4096, 8), 0.5, flops=0.5e-3 * 1.4e15 * 0.5)          # GEMMs at half of peak
    learned = white_search(model, 8, hw, topk=3, db=db, comm=comm)
    tp_before = base[0].config.tp
    assert learned[0].config.tp <= tp_before and learned[0].step_ms != base[0].step_ms
    assert learned[0].config.tp < 8                              # expensive tensor-parallel traffic pushes the choice away from TP8


def test_stage_1_prune_keeps_minimal_recompute_and_drops_oversized():
    from mindspeed_b200.auto_settings.cost_model import memory_gib
    from mindspeed_b200.auto_settings.hardware import Hardware
    from mindspeed_b200.auto_settings.search_space import ModelDesc, build_search_space, stage_1_prune
    model = ModelDesc(32, 4096, 14336, 32, 8, 128256, 8192, 64)
    space = build_search_space(model, 8)
    kept = stage_1_prune(space, model, memory_gib, Hardware().hbm_gib)
    assert 0 < len(kept) < len(space)
    keys = [(c.tp, c.cp, c.pp, c.dp, c.ep, c.mbs) for c in kept]
    assert len(keys) == len(set(keys))                           # one recompute level per layout: the smallest that fits
    assert all(memory_gib(model, c)["total"] <= Hardware().hbm_gib for c in kept)


def test_learn_from_profile_feeds_db_and_lines():
    from mindspeed_b200.auto_settings.comm_predictors import CommPredictors
    from mindspeed_b200.auto_settings.cost_model import learn_from_profile
    from mindspeed_b200.auto_settings.hardware import Hardware
    from mindspeed_b200.auto_settings.operator_db import OperatorDB
    from mindspeed_b200.auto_settings.profiling_parse import summarize
    from mindspeed_b200.auto_settings.search_space import ModelDesc, SearchConfig
    hw, db = Hardware(), OperatorDB()
    comm = CommPredictors(hw)
    model = ModelDesc(2, 1024, 4096, 8, 8, 32000, 2048, 8, num_experts=8, moe_topk=2)
    cfg = SearchConfig(tp=1, cp=1, pp=1, dp=8, ep=8, mbs=1)
    learn_from_profile(summarize(_trace()), model, cfg, hw, db, comm)
    assert db.exact("gemm", (2048, 1024, 1)) is not None and db.exact("attention", (2048, 2048, 8)) is not None
    assert len(comm.total["ep"].samples) == 1 and comm.exposed["ep"].samples[0][1] < comm.total["ep"].samples[0][1]


def _ootb(rank, world, save, env):
    import io
    import os
    import sys
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    os.environ[env] = "TRUE"
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + ["--pipeline-model-parallel-size", str(world), "--profile-save-path", save])
    return hist


def test_launch_can_report_its_arguments_and_parameters_without_training(tmp_path):
    """OOTB_OPTIMIZER_PARSE_ARGS / OOTB_OPTIMIZER_PARSE_MODEL: the launcher writes what it resolved and stops."""
    import json
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    d = str(tmp_path)
    assert run_distributed(_ootb, 2, d, "OOTB_OPTIMIZER_PARSE_ARGS") == [[], []]
    a = json.load(open(os.path.join(d, "auto_settings_args.json")))
    assert a["pipeline_model_parallel_size"] == 2 and a["hidden_size"] == 64 and a["data_parallel_size"] == 1
    assert run_distributed(_ootb, 2, d, "OOTB_OPTIMIZER_PARSE_MODEL") == [[], []]
    p0 = json.load(open(os.path.join(d, "model_params_pp0.json")))
    p1 = json.load(open(os.path.join(d, "model_params_pp1.json")))
    n0, n1 = {r["name"] for r in p0["parameters"]}, {r["name"] for r in p1["parameters"]}
    assert "embedding.word_embeddings.weight" in n0 and "output_layer.weight" in n1 and "output_layer.weight" not in n0
    qkv = next(r for r in p0["parameters"] if r["name"].endswith("linear_qkv.weight"))
    assert qkv["tensor_parallel"] and qkv["partition_dim"] == 0 and qkv["numel"] == qkv["shape"][0] * qkv["shape"][1]
    assert p0["total_numel"] == sum(r["numel"] for r in p0["parameters"])
