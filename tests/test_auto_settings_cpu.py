def _llama():
    from mindspeed_b200.auto_settings import ModelDesc
    return ModelDesc(32, 4096, 14336, 32, 8, 128256, 8192, 64)


def test_search_space_rules():
    from mindspeed_b200.auto_settings import build_search_space
    sp = build_search_space(_llama(), 8)
    assert sp and all(c.tp * c.cp * c.pp * c.dp == 8 for c in sp)
    assert all(32 % c.pp == 0 and 8 % c.tp == 0 for c in sp)             # layers % pp, kv groups % tp
    assert all(8192 // c.cp >= 4096 or c.cp == 1 for c in sp)            # minimum sequence per cp rank
    assert all(64 % (c.dp * c.mbs) == 0 for c in sp)
    assert not any(c.ep > 1 for c in sp)                                 # dense model: no expert parallelism


def test_memory_model_orders_configs_sensibly():
    from mindspeed_b200.auto_settings import Hardware, SearchConfig, memory_gib
    m = _llama()
    tp8 = memory_gib(m, SearchConfig(tp=8, dp=1))["total"]
    tp1 = memory_gib(m, SearchConfig(tp=1, dp=8, use_distributed_optimizer=False))["total"]
    tp1_zero = memory_gib(m, SearchConfig(tp=1, dp=8, use_distributed_optimizer=True))["total"]
    assert tp8 < 60 and tp1 > Hardware().hbm_gib and tp1_zero < tp1
    full = memory_gib(m, SearchConfig(tp=1, dp=8, recompute_layers=32))["activations"]
    none = memory_gib(m, SearchConfig(tp=1, dp=8, recompute_layers=0))["activations"]
    assert full < 0.3 * none


def test_white_and_black_search():
    from mindspeed_b200.auto_settings import Hardware, black_search, white_search
    hw = Hardware()
    best = white_search(_llama(), 8, hw, topk=3)
    assert len(best) == 3 and all(e.fits for e in best)
    assert best[0].step_ms <= best[1].step_ms <= best[2].step_ms
    # fused TP communication must make TP>1 cheaper than the unfused estimate of the same config
    from mindspeed_b200.auto_settings import SearchConfig, step_ms
    a = step_ms(_llama(), SearchConfig(tp=8, fused_tp_comm=True), hw)["total_ms"]
    b = step_ms(_llama(), SearchConfig(tp=8, fused_tp_comm=False), hw)["total_ms"]
    assert a < b
    calls = []

    def fake_run(cfg):
        calls.append(cfg)
        return None if cfg.tp == 8 else 1000.0 / cfg.dp + cfg.pp      # pretend TP8 runs out of memory
    got = black_search(_llama(), 8, hw, fake_run, topk=2, budget=6)
    assert len(calls) == 6 and all(e.config.tp != 8 for e in got) and got[0].step_ms <= got[-1].step_ms


def test_executor_command_line():
    from mindspeed_b200.auto_settings import SearchConfig
    from mindspeed_b200.auto_settings.executor import TorchrunExecutor
    ex = TorchrunExecutor(["--num-layers", "2"], 4)
    cmd = ex.command(SearchConfig(tp=2, dp=2, recompute_layers=1))
    assert "--nproc-per-node" in cmd and "--tensor-model-parallel-size" in cmd and "--use-fused-tp-comm" in cmd
    assert "--master-addr" in cmd and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
