"""fp8 recipes and TE-compatible modules on CPU (the fp8 arithmetic is evaluated in fp32 from real fp8 casts)."""
import pytest
import torch
import torch.nn as nn


def _cfg(**kw):
    from mindspeed_b200.config import TransformerConfig
    return TransformerConfig(num_layers=1, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, use_cpu_initialization=True,
                             add_bias_linear=False, normalization="RMSNorm", hidden_dropout=0.0, attention_dropout=0.0, **kw)


@pytest.mark.parametrize("name,tol", [("tensorwise", 0.06), ("delayed", 0.06), ("blockwise", 0.05), ("mxfp8", 0.05)])
def test_recipe_round_trip_error(name, tol):
    from mindspeed_b200.models import te_compat as TE
    torch.manual_seed(0)
    r = TE.RECIPES[name]()
    x = torch.randn(64, 256) * torch.logspace(-2, 2, 64).unsqueeze(1)     # rows of very different magnitude
    state = {}
    y = r.round_trip(x, "inputs", state)
    rel = ((y - x).norm(dim=1) / x.norm(dim=1))
    if name in ("blockwise", "mxfp8"):
        assert rel.max() < tol                      # block scales follow each row's magnitude
    else:
        assert rel[-8:].max() < tol                 # per-tensor scale: only the large rows keep precision
        assert rel[:4].min() > rel[-4:].max()       # ... and the small rows lose it (underflow) - what block scaling fixes
    g = r.round_trip(x, "grads", state)
    assert r.dtype_for("grads") == torch.float8_e5m2 and ((g - x).norm() / x.norm()) < 0.12


def test_delayed_scaling_uses_history():
    from mindspeed_b200.models import te_compat as TE
    r = TE.DelayedScaling(amax_history_len=3)
    st = {}
    small = torch.full((4, 4), 1.0)
    big = torch.full((4, 4), 1000.0)
    r.round_trip(small, "inputs", st)
    out = r.round_trip(big, "inputs", st)           # scale still comes from the history (amax 1): the big tensor saturates
    assert out.max() <= 448.0 + 1e-3
    out2 = r.round_trip(big, "inputs", st)          # now the history knows about 1000
    assert abs(out2.max().item() - 1000.0) / 1000.0 < 0.07
    for _ in range(3):
        r.round_trip(small, "inputs", st)
    assert st["inputs"] == [1.0, 1.0, 1.0]


@pytest.mark.parametrize("recipe", ["blockwise", "tensorwise", "mxfp8"])
def test_te_linears_under_autocast(recipe):
    from mindspeed_b200.models import te_compat as TE
    cfg = _cfg()
    torch.manual_seed(1)
    col = TE.TEColumnParallelLinear(256, 512, config=cfg, init_method=cfg.init_method, bias=False)
    row = TE.TERowParallelLinear(512, 256, config=cfg, init_method=cfg.init_method, bias=False)
    x = torch.randn(8, 2, 256, requires_grad=True)
    y_ref, _ = row(torch.tanh(col(x)[0]))
    g = torch.randn_like(y_ref)
    y_ref.backward(g)
    gx_ref, gw_ref = x.grad.clone(), col.weight.grad.clone()
    x.grad = None
    col.weight.grad = None
    row.weight.grad = None
    with TE.fp8_autocast(True, TE.RECIPES[recipe]()):
        assert TE.fp8_enabled()
        y, _ = row(torch.tanh(col(x)[0]))
    assert not TE.fp8_enabled()
    y.backward(g)
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert 1e-4 < rel(y, y_ref) < 0.1
    assert rel(x.grad, gx_ref) < 0.15 and rel(col.weight.grad, gw_ref) < 0.15
    if recipe == "blockwise":
        assert "wq" in col._fp8_wcache
        TE.clear_fp8_weight_cache()
        assert not col._fp8_wcache


def test_layernorm_linear_grouped_linear_and_quantize_linears():
    from mindspeed_b200.models import te_compat as TE
    cfg = _cfg()
    torch.manual_seed(2)
    ln = TE.TELayerNormColumnParallelLinear(256, 384, config=cfg, init_method=cfg.init_method, bias=False)
    x = torch.randn(5, 3, 256)
    y, b = ln(x)
    assert y.shape == (5, 3, 384) and b is None
    ln.return_layernorm_output = True
    (y2, n), _ = ln(x)
    assert torch.allclose(y, y2) and n.shape == x.shape
    gl = TE.TEGroupedLinear(3, 256, 128, config=cfg)
    rows = torch.randn(10, 256)
    out, _ = gl(rows, [4, 0, 6])
    ref = torch.cat([rows[:4] @ gl.weight[0].t(), rows[4:] @ gl.weight[2].t()])
    assert torch.allclose(out, ref, atol=1e-4)
    with torch.no_grad(), TE.fp8_autocast(True, TE.BlockwiseScaling()):
        out8, _ = gl(rows, [4, 0, 6])
    assert ((out8 - ref).norm() / ref.norm()) < 0.08
    net = nn.Sequential(nn.Linear(256, 256), nn.ReLU(), nn.Linear(256, 128))
    assert TE.quantize_linears(net, "blockwise") == 2 and isinstance(net[0], TE.Fp8Linear)
    z = net(torch.randn(4, 256))
    z.sum().backward()
    assert net[0].weight.grad is not None


def test_online_comparison_records_errors_and_stops_on_a_bad_result():
    import torch
    from mindspeed_b200.models import te_compat as TE
    torch.manual_seed(0)
    lin = TE.Fp8Linear(torch.nn.Linear(64, 32, bias=False), TE.MXFP8Scaling())
    x = torch.randn(16, 64)
    try:
        for with_cpu in (False, True):
            TE.OnlineComparison.configure(with_bf16=not with_cpu, with_cpu=with_cpu)
            lin(x)
            rec = TE.OnlineComparison.records[-1]
            assert rec["reference"] == ("cpu" if with_cpu else "bf16") and 1e-4 < rec["rel_err"] < 0.1
            assert rec["shape"] == ((16, 64), (32, 64))
        TE.OnlineComparison.configure(with_bf16=True, limit=1e-6)       # fp8 cannot meet this: the run stops
        import pytest
        with pytest.raises(RuntimeError, match="deviates from the bf16 reference"):
            lin(x)
    finally:
        TE.OnlineComparison.configure()
    assert TE.OnlineComparison.mode is None
    lin(x)
    assert TE.OnlineComparison.records == []
