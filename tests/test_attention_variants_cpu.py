"""ALiBi: the blocked slope-based attention against attention with the dense bias tensor, and a GPT model trained with it."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from mindspeed_b200.models.attention_masks import alibi_bias, alibi_slopes
from mindspeed_b200.ops.attention import alibi_attention


def _dense(q, k, v, bias, causal, scale):
    sq, b, n, d = q.shape
    sk = k.shape[0]
    rep = n // k.shape[2]
    kf = k.permute(1, 2, 0, 3).double().repeat_interleave(rep, 1)
    vf = v.permute(1, 2, 0, 3).double().repeat_interleave(rep, 1)
    s = torch.matmul(q.permute(1, 2, 0, 3).double(), kf.transpose(-1, -2)) * scale + bias.double().unsqueeze(0)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(sq, sk, dtype=torch.bool), 1 + sk - sq), float("-inf"))
    return torch.matmul(torch.softmax(s, -1), vf).permute(2, 0, 1, 3)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("heads,groups", [(4, 4), (6, 2)])
def test_blocked_slope_attention_equals_dense_bias_attention(causal, heads, groups):
    g = torch.Generator().manual_seed(0)
    S, B, d = 37, 2, 8
    q = torch.randn(S, B, heads, d, generator=g, requires_grad=True)
    k = torch.randn(S, B, groups, d, generator=g, requires_grad=True)
    v = torch.randn(S, B, groups, d, generator=g, requires_grad=True)
    sl = alibi_slopes(heads)
    i, j = torch.arange(S).view(S, 1), torch.arange(S).view(1, S)
    for mode, signed, bias in ((0, False, alibi_bias(heads, S, S, symmetric=True)),
                               (2, False, -sl.view(-1, 1, 1) * (i - j).abs()),
                               (3, False, -sl.view(-1, 1, 1) * (i - j).abs().float().sqrt()),
                               (0, True, sl.view(-1, 1, 1) * (j - i))):
        out = alibi_attention(q, k, v, sl, causal=causal, mode=mode, signed=signed, block=16)
        ref = _dense(q, k, v, bias, causal, 1 / math.sqrt(d))
        assert torch.allclose(out.double(), ref, atol=1e-5), (mode, signed)
        go = torch.randn(out.shape, generator=g)
        for a, r in zip(torch.autograd.grad(out, (q, k, v), go), torch.autograd.grad(ref, (q, k, v), go.double())):
            assert torch.allclose(a.double(), r.double(), atol=1e-5), (mode, signed)
    if causal:                # under a causal mask the signed form is the default one
        a = alibi_attention(q, k, v, sl, causal=True, signed=True)
        assert torch.allclose(a, alibi_attention(q, k, v, sl, causal=True), atol=1e-6)


def _train(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    base = [a for a in BASE]
    i = base.index("--position-embedding-type")
    base[i + 1] = "alibi"
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=base + list(extra))
    return [h["lm loss"] for h in hist]


def test_gpt_with_alibi_trains_the_same_under_tensor_parallelism():
    from dist_utils import run_distributed
    one = run_distributed(_train, 1, ["--alibi-fusion-attn-type", "2"])[0]
    dense = run_distributed(_train, 1, ["--alibi-fusion-attn-type", "0", "--alibi-diagonal-opposite"])[0]
    assert one == pytest.approx(dense, abs=1e-5)                    # causal model: same function
    sq = run_distributed(_train, 1, ["--alibi-fusion-attn-type", "3"])[0]
    assert sq != pytest.approx(one, abs=1e-6)
    tp = run_distributed(_train, 2, ["--alibi-fusion-attn-type", "2", "--tensor-model-parallel-size", "2"])[0]
    assert tp == pytest.approx(one, abs=2e-4)                        # each rank takes the slopes of its own heads


def test_flags_validate():
    from mindspeed_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128"]
    a = validate_args(parse_args(args_list=base + ["--position-embedding-type", "alibi", "--alibi-fusion-attn-type", "2"]))
    from mindspeed_b200.training.arguments import core_transformer_config_from_args
    cfg = core_transformer_config_from_args(a)
    assert cfg.position_embedding_type == "alibi" and cfg.alibi_fusion_attn_type == 2
    with pytest.raises(AssertionError, match="position-embedding-type alibi"):
        validate_args(parse_args(args_list=base + ["--alibi-fusion-attn-type", "2"]))
    with pytest.raises(AssertionError, match="linear bias"):
        validate_args(parse_args(args_list=base + ["--position-embedding-type", "alibi", "--alibi-fusion-attn-type", "3",
                                                   "--alibi-diagonal-opposite"]))


@pytest.mark.parametrize("pre,nxt,sk", [(5, 0, 40), (3, 2, 40), (100, 0, 40), (4, 0, 52), (0, 0, 40)])
def test_sliding_window_attention_equals_band_masked_attention(pre, nxt, sk):
    from mindspeed_b200.ops.attention import attention_ref, band_attention
    g = torch.Generator().manual_seed(1)
    sq, B, n, d = 40, 2, 4, 8
    q = torch.randn(sq, B, n, d, generator=g, requires_grad=True)
    k = torch.randn(sk, B, 2, d, generator=g, requires_grad=True)
    v = torch.randn(sk, B, 2, d, generator=g, requires_grad=True)
    i = torch.arange(sq).view(sq, 1) + (sk - sq)
    j = torch.arange(sk).view(1, sk)
    hidden = (j < i - pre) | (j > i + nxt)
    ref = attention_ref(q, k, v, causal=False, mask=hidden.view(1, 1, sq, sk))
    out = band_attention(q, k, v, pre, nxt, block=16)
    assert torch.allclose(out, ref, atol=1e-5)
    go = torch.randn(out.shape, generator=g)
    for a, b in zip(torch.autograd.grad(out, (q, k, v), go), torch.autograd.grad(ref, (q, k, v), go)):
        assert torch.allclose(a, b, atol=1e-5)


def _train_window(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.ops import attention as OA
    from mindspeed_b200.training import pretrain
    calls = []
    orig = OA.band_attention
    OA.band_attention = lambda q, k, v, pre, nxt, **kw: (calls.append((pre, nxt)), orig(q, k, v, pre, nxt, **kw))[1]
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + list(extra))
    OA.band_attention = orig
    return [h["lm loss"] for h in hist], sorted(set(calls))


def test_window_flags_select_sliding_window_attention():
    from dist_utils import run_distributed
    plain, c0 = run_distributed(_train_window, 1, [])[0]
    assert c0 == []                                                   # default bounds: plain causal attention
    a, ca = run_distributed(_train_window, 1, ["--pre-tockens", "8", "--sparse-mode", "4"])[0]
    b, cb = run_distributed(_train_window, 1, ["--window-size", "8,0"])[0]
    assert ca == [(8, 0)] and cb == [(8, 0)] and a == pytest.approx(b, abs=1e-6) and a != pytest.approx(plain, abs=1e-6)
    c, cc = run_distributed(_train_window, 1, ["--pre-tockens", "8", "--sparse-mode", "2"])[0]
    assert cc == [] and c == pytest.approx(plain, abs=1e-6)           # mode 2: causal, the bounds are not used
    d, cd = run_distributed(_train_window, 1, ["--window-size", "64,0"])[0]
    assert cd == [] and d == pytest.approx(plain, abs=1e-6)           # a window that covers the sequence
