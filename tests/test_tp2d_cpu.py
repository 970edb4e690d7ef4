"""2-D tensor parallel linear and norms on 4 gloo ranks (x=2, y=2) against the dense computation."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _run(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.tp2d import ParallelLinear2D, RMSNorm2D
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(tensor_model_parallel_size=4, tp_2d=True, tp_x=2, tp_y=2)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True, optimization_level=0)
    gx, gy = ps.get_tp_x_group(), ps.get_tp_y_group()
    xi, yi = ps.get_tp_x_rank(), ps.get_tp_y_rank()
    S, B, H, E = 16, 2, 32, 48
    g = torch.Generator().manual_seed(0)
    X = torch.randn(S, B, H, generator=g)
    W1 = torch.randn(E, H, generator=g) * 0.1
    W2 = torch.randn(H, E, generator=g) * 0.1
    Wgt = torch.randn(S, B, H, generator=g)

    def init(w):
        return lambda t: t.copy_(w)
    l1 = ParallelLinear2D(H, E, config=cfg, init_method=init(W1), ag_group=gx, rs_group=gy)   # seq over x, hidden over y
    l2 = ParallelLinear2D(E, H, config=cfg, init_method=init(W2), ag_group=gy, rs_group=gx)   # roles swapped
    norm = RMSNorm2D(H, 1e-5, cfg, group=gy)
    xl = X.chunk(2, 0)[xi].chunk(2, 2)[yi].clone().requires_grad_(True)
    h, _ = l1(norm(xl))
    out, _ = l2(torch.tanh(h))
    wl = Wgt.chunk(2, 0)[xi].chunk(2, 2)[yi]
    (out * wl).sum().backward()
    # dense reference
    Xr = X.clone().requires_grad_(True)
    W1r, W2r = W1.clone().requires_grad_(True), W2.clone().requires_grad_(True)
    nr = Xr * torch.rsqrt(Xr.pow(2).mean(-1, keepdim=True) + 1e-5)
    ref = torch.tanh(nr @ W1r.t()) @ W2r.t()
    (ref * Wgt).sum().backward()
    res = {"out": (out.detach() - ref.detach().chunk(2, 0)[xi].chunk(2, 2)[yi]).abs().max().item(),
           "dx": (xl.grad - Xr.grad.chunk(2, 0)[xi].chunk(2, 2)[yi]).abs().max().item(),
           "dw1": (l1.weight.grad - W1r.grad.chunk(2, 0)[xi].chunk(2, 1)[yi]).abs().max().item(),
           "dw2": (l2.weight.grad - W2r.grad.chunk(2, 0)[yi].chunk(2, 1)[xi]).abs().max().item()}
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return res


def test_tp2d_linear_and_norm_match_dense():
    for r in run_distributed(_run, 4):
        for k, v in r.items():
            assert v < 1e-4, (k, v, r)


def _run_block(rank, world):
    import torch.distributed as dist
    import torch.nn.functional as F
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.ops.rope import apply_rope_ref
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.tp2d import MLP2D, RMSNorm2D, SelfAttention2D, from_2d_layout, to_2d_layout
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(tensor_model_parallel_size=4, tp_2d=True, tp_x=2, tp_y=2)
    S, B, H, NH, NG, D, FF = 16, 2, 32, 4, 2, 8, 48
    g = torch.Generator().manual_seed(1)
    Wqkv = torch.randn((NH + 2 * NG) * D, H, generator=g) * 0.2
    Wproj = torch.randn(H, NH * D, generator=g) * 0.2
    Wfc1 = torch.randn(2 * FF, H, generator=g) * 0.2
    Wfc2 = torch.randn(H, FF, generator=g) * 0.2
    X = torch.randn(S, B, H, generator=g)
    Wgt = torch.randn(S, B, H, generator=g)
    ang = torch.outer(torch.arange(S).float(), 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D)))
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos(), emb.sin()
    it = iter([Wqkv, Wproj, Wfc1, Wfc2])

    def init_from_list(t):
        return t.copy_(next(it))
    cfg = TransformerConfig(num_layers=1, hidden_size=H, num_attention_heads=NH, num_query_groups=NG, kv_channels=D,
                            ffn_hidden_size=FF, gated_linear_unit=True, activation_func=F.silu, add_bias_linear=False,
                            use_cpu_initialization=True, optimization_level=0, normalization="RMSNorm")
    cfg.init_method = init_from_list
    cfg.output_layer_init_method = init_from_list
    attn = SelfAttention2D(cfg)           # consumes Wqkv, Wproj
    mlp = MLP2D(cfg)                      # consumes Wfc1, Wfc2
    n1, n2 = RMSNorm2D(H, 1e-5, cfg), RMSNorm2D(H, 1e-5, cfg)
    Xl = X.clone().requires_grad_(True)
    h = to_2d_layout(Xl)
    a, _ = attn(n1(h), rotary_pos_emb=(cos, sin))
    h = h + a
    m, _ = mlp(n2(h))
    h = h + m
    out = from_2d_layout(h)
    (out * Wgt).sum().backward()          # every rank uses the gathered output: the gradients add up over the 4 ranks
    # dense oracle
    Xr = X.clone().requires_grad_(True)
    rms = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5)
    qkv = (rms(Xr) @ Wqkv.t()).view(S, B, NG, NH // NG + 2, D)
    q = qkv[:, :, :, :NH // NG].reshape(S, B, NH, D)
    k, v = qkv[:, :, :, NH // NG], qkv[:, :, :, NH // NG + 1]
    q, k = apply_rope_ref(q, cos, sin), apply_rope_ref(k, cos, sin)
    ctx = attention_ref(q, k, v, causal=True)
    hr = Xr + ctx.reshape(S, B, NH * D) @ Wproj.t()
    f1 = rms(hr) @ Wfc1.t()
    hr = hr + (F.silu(f1[..., :FF]) * f1[..., FF:]) @ Wfc2.t()
    (hr * Wgt).sum().backward()
    res = {"out": (out.detach() - hr.detach()).abs().max().item(), "dx": (Xl.grad - 4 * Xr.grad).abs().max().item()}
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return res


def test_tp2d_attention_and_mlp_block_matches_dense():
    """Norm -> attention -> norm -> gated MLP with [s/x, b, h/y] activations between the blocks, heads split over x and the
    sequence over y inside attention (K / V gathered over y), against the dense block."""
    for r in run_distributed(_run_block, 4):
        for k, v in r.items():
            assert v < 2e-4, (k, v, r)


def _train_2d(rank, world, prefix, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + ["--group-query-attention", "--num-query-groups", "2", "--train-iters", "10", "--lr", "1e-2",
                                          "--data-path", prefix, "--split", "100,0,0"] + list(extra))
    return [h["lm loss"] for h in hist]


def test_gpt_trains_with_2d_tensor_parallel(tmp_path):
    """The GPT model built from 2-D blocks (--tp-2d, x = 2, y = 2) learns a small corpus about as fast as the one-rank
    model; every tensor-parallel rank reports the same loss."""
    from test_gpt_dataset_cpu import _corpus
    prefix = str(tmp_path / "c")
    _corpus(prefix, n_docs=60, vocab=100)
    ref = run_distributed(_train_2d, 1, prefix, [])[0]
    res = run_distributed(_train_2d, 4, prefix, ["--tensor-model-parallel-size", "4", "--tp-2d", "--tp-x", "2", "--tp-y", "2"])
    assert all(r == res[0] for r in res)
    assert ref[-1] < ref[0] - 0.1 and res[0][-1] < res[0][0] - 0.1, (ref, res[0])
    assert abs(res[0][0] - ref[0]) < 0.1                      # same model size and data: the first loss is ln(vocab)-ish for both
    assert abs(res[0][-1] - ref[-1]) < 0.5 * (ref[0] - ref[-1])
