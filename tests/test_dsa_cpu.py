"""DeepSeek sparse attention: the selected-key attention ops against dense masked attention, the absorbed (latent) form
against the per-head form, and the MLA layer with its lightning indexer and KL loss."""
import math

import pytest
import torch

from mindspeed_b200.ops import lightning_indexer as LI
from mindspeed_b200.ops import sparse_attention as SA


def _dense_masked(q, k, v, idx, scale):
    B, T, H, d = q.shape
    S = k.shape[1]
    mask = LI.sparse_attention_mask(idx, S)                                     # [B, T, S] additive
    s = torch.einsum("bthd,bshd->bhts", q.double(), k.double()) * scale + mask.unsqueeze(1).double()
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhts,bshd->bthd", p, v.double()), p.mean(dim=1)


def _random_selection(B, T, S, K, g):
    idx = torch.full((B, T, K), -1, dtype=torch.long)
    for b in range(B):
        for t in range(T):
            vis = t + 1 + (S - T)
            n = min(K, vis)
            idx[b, t, :n] = torch.randperm(vis, generator=g)[:n]
    return idx


def test_sparse_attention_matches_dense_attention_under_the_selection_mask():
    g = torch.Generator().manual_seed(0)
    B, T, H, d, dv, K = 2, 24, 3, 16, 8, 5
    q, k, v = torch.randn(B, T, H, d, generator=g), torch.randn(B, T, H, d, generator=g), torch.randn(B, T, H, dv, generator=g)
    idx = _random_selection(B, T, T, K, g)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    o, p = SA.sparse_attention(q, k, v, idx, 0.25, block=7)
    ro, rp = _dense_masked(q, k, v, idx, 0.25)
    assert torch.allclose(o.double(), ro, atol=1e-5)
    got = torch.zeros(B, T, T + 1).scatter_(2, idx.masked_fill(idx < 0, T), p)[..., :T]
    assert torch.allclose(got.double(), rp, atol=1e-6)
    go = torch.randn(o.shape, generator=g)
    g1 = torch.autograd.grad(o, (q, k, v), go)
    g2 = torch.autograd.grad(ro, (q, k, v), go.double())
    for a, b in zip(g1, g2):
        assert torch.allclose(a.double(), b.double(), atol=1e-5)


def test_latent_form_equals_per_head_form():
    g = torch.Generator().manual_seed(1)
    B, T, H, dn, dr, dv, r, K = 2, 20, 4, 8, 4, 6, 12, 6
    q_nope, q_pe = torch.randn(B, T, H, dn, generator=g), torch.randn(B, T, H, dr, generator=g)
    kv, k_pe = torch.randn(B, T, r, generator=g), torch.randn(B, T, dr, generator=g)
    w_uk, w_uv = torch.randn(H, dn, r, generator=g) / math.sqrt(r), torch.randn(H, dv, r, generator=g) / math.sqrt(r)
    idx = _random_selection(B, T, T, K, g)
    k_nope = torch.einsum("bsr,hdr->bshd", kv, w_uk)
    v = torch.einsum("bsr,hvr->bshv", kv, w_uv)
    qf = torch.cat((q_nope, q_pe), dim=-1)
    kf = torch.cat((k_nope, k_pe.unsqueeze(2).expand(B, T, H, dr)), dim=-1)
    o1, p1 = SA.sparse_attention(qf, kf, v, idx, 0.3)
    q_lat = torch.einsum("bthd,hdr->bthr", q_nope, w_uk)
    ol, p2 = SA.sparse_latent_attention(q_lat, q_pe, kv, k_pe, idx, 0.3, block=8)
    o2 = torch.einsum("bthr,hvr->bthv", ol, w_uv)
    assert torch.allclose(o1, o2, atol=1e-5)
    assert torch.allclose(p1, p2, atol=1e-6)


def test_selected_kl_loss_is_zero_at_the_target_and_has_finite_gradients():
    g = torch.Generator().manual_seed(2)
    B, T, K = 2, 10, 4
    idx = _random_selection(B, T, T, K, g)
    sc = torch.randn(B, T, T, generator=g)
    sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf")).requires_grad_(True)
    valid = idx >= 0
    tgt = torch.softmax(torch.gather(sc.detach(), 2, idx.clamp_min(0)).masked_fill(~valid, float("-inf")), dim=-1)
    assert float(SA.selected_kl_loss(sc, idx, tgt)) < 1e-6
    other = torch.rand(B, T, K, generator=g) * valid
    for red, div in (("sum", 1), ("mean", B * T), ("batchmean", B * T)):
        loss = SA.selected_kl_loss(sc, idx, other, red)
        assert float(loss) > 0
        if red == "sum":
            total = float(loss)
        assert abs(float(loss) - total / div) < 1e-5
    (gr,) = torch.autograd.grad(SA.selected_kl_loss(sc, idx, other), sc)
    assert torch.isfinite(gr).all() and gr.abs().sum() > 0


def _mla_config(**kw):
    from mindspeed_b200.config import MLATransformerConfig
    base = dict(num_layers=1, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, q_lora_rank=32, kv_lora_rank=24,
                qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16, rope_type="rope", rotary_scaling_factor=1,
                params_dtype=torch.float32, use_cpu_initialization=True, optimization_level=0, qk_layernorm=True,
                normalization="RMSNorm", add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0,
                experimental_attention_variant="dsa", dsa_indexer_n_heads=2, dsa_indexer_head_dim=16)
    base.update(kw)
    return MLATransformerConfig(**base)


def _rope(S, d):
    inv = 1.0 / (10000 ** (torch.arange(0, d, 2).float() / d))
    ang = torch.outer(torch.arange(S).float(), inv)
    emb = torch.cat((ang, ang), dim=-1).view(S, 1, 1, d)
    return emb.cos(), emb.sin()


@pytest.fixture
def single_rank():
    from mindspeed_b200.parallel import parallel_state as ps
    import torch.distributed as dist
    import os
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", str(__import__("dist_utils")._free_port()))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1, 1)
    from mindspeed_b200.parallel.random import model_parallel_cuda_manual_seed
    torch.manual_seed(5)
    yield
    ps.destroy_model_parallel()


def test_mla_layer_with_full_selection_equals_dense_mla_and_absorb_changes_nothing(single_rank):
    from mindspeed_b200.models.attention import MLASelfAttention
    from mindspeed_b200.models import dsa as D
    S, B = 12, 2
    rope = _rope(S, 8)
    x = torch.randn(S, B, 64)
    dense = MLASelfAttention(_mla_config(experimental_attention_variant=None))
    full = MLASelfAttention(_mla_config(dsa_indexer_topk=S))
    full.load_state_dict(dense.state_dict(), strict=False)
    yd, _ = dense(x, rotary_pos_emb=rope)
    yf, _ = full(x, rotary_pos_emb=rope)
    assert torch.allclose(yd, yf, atol=1e-5)

    sparse = MLASelfAttention(_mla_config(dsa_indexer_topk=4))
    absorb = MLASelfAttention(_mla_config(dsa_indexer_topk=4, use_dsa_absorb=True))
    absorb.load_state_dict(sparse.state_dict())
    xs = x.clone().requires_grad_(True)
    xa = x.clone().requires_grad_(True)
    ys, _ = sparse(xs, rotary_pos_emb=rope)
    l1 = D.dsa_indexer_losses()[1]
    ya, _ = absorb(xa, rotary_pos_emb=rope)
    assert torch.allclose(ys, ya, atol=1e-5)
    assert not torch.allclose(ys, yd, atol=1e-3)                  # four keys per query is a different function
    assert torch.allclose(l1, D.dsa_indexer_losses()[1], atol=1e-6) and float(l1) > 0
    ys.sum().backward(); ya.sum().backward()
    assert torch.allclose(xs.grad, xa.grad, atol=1e-5)
    for (n, p), (_, q) in zip(sparse.named_parameters(), absorb.named_parameters()):
        assert p.grad is not None, n
        assert torch.allclose(p.grad, q.grad, atol=1e-4), n
    # the indexer is trained by the KL loss alone: the main model gets no gradient through the selection
    assert sparse.indexer.wq.grad.abs().sum() > 0


def test_indexer_learns_the_attention_distribution(single_rank):
    from mindspeed_b200.models.attention import MLASelfAttention
    from mindspeed_b200.models import dsa as D
    S, B = 16, 2
    rope = _rope(S, 8)
    layer = MLASelfAttention(_mla_config(dsa_indexer_topk=S))      # every visible key selected: pure indexer fitting
    opt = torch.optim.Adam(layer.indexer.parameters(), lr=2e-2)
    x = torch.randn(S, B, 64)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        y, _ = layer(x, rotary_pos_emb=rope)
        (y.sum() * 0).backward()                                   # only the attached KL loss contributes
        losses.append(float(D.dsa_indexer_losses()[1]))
        opt.step()
    assert losses[-1] < 0.5 * losses[0]


def test_recomputed_up_projections_change_nothing(single_rank):
    from mindspeed_b200.models.attention import MLASelfAttention
    S, B = 12, 2
    rope = _rope(S, 8)
    a = MLASelfAttention(_mla_config(experimental_attention_variant=None))
    b = MLASelfAttention(_mla_config(experimental_attention_variant=None, recompute_mla_up_proj=True))
    b.load_state_dict(a.state_dict())
    x1 = torch.randn(S, B, 64, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_(True)
    y1, _ = a(x1, rotary_pos_emb=rope)
    y2, _ = b(x2, rotary_pos_emb=rope)
    assert torch.allclose(y1, y2, atol=1e-6)
    y1.pow(2).sum().backward(); y2.pow(2).sum().backward()
    assert torch.allclose(x1.grad, x2.grad, atol=1e-6)
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5), n


def test_flags_validate():
    from mindspeed_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128"]
    mla = ["--multi-head-latent-attention", "--qk-layernorm", "--experimental-attention-variant", "dsa"]
    a = validate_args(parse_args(args_list=base + mla + ["--use-dsa-absorb", "--dsa-indexer-topk", "8"]))
    from mindspeed_b200.training.arguments import core_transformer_config_from_args
    cfg = core_transformer_config_from_args(a)
    assert cfg.experimental_attention_variant == "dsa" and cfg.use_dsa_absorb and cfg.dsa_indexer_topk == 8
    with pytest.raises(AssertionError, match="qk-layernorm"):
        validate_args(parse_args(args_list=base + ["--multi-head-latent-attention", "--experimental-attention-variant", "dsa"]))
    with pytest.raises(AssertionError, match="come as a set"):
        validate_args(parse_args(args_list=base + mla + ["--use-fused-lightning-indexer"]))
    with pytest.raises(AssertionError, match="experimental-attention-variant dsa"):
        validate_args(parse_args(args_list=base + ["--use-dsa-absorb"]))


MLA = ["--multi-head-latent-attention", "--qk-layernorm", "--q-lora-rank", "32", "--kv-lora-rank", "24", "--qk-nope-head-dim", "16",
       "--qk-rope-head-dim", "8", "--v-head-dim", "16", "--train-iters", "3", "--global-batch-size", "4", "--lr", "3e-3"]
DSA = ["--experimental-attention-variant", "dsa", "--dsa-indexer-n-heads", "2", "--dsa-indexer-head-dim", "16",
       "--dsa-indexer-topk", "8"]


def _train(rank, world, extra):
    import io
    import os
    import sys
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.models import dsa as D
    from mindspeed_b200.training import pretrain
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + MLA + list(extra))
    return [h["lm loss"] for h in hist], {k: float(v) for k, v in D.dsa_indexer_losses().items()}


def test_gpt_with_latent_attention_trains_dense_and_sparse_also_under_tensor_parallelism():
    from dist_utils import run_distributed
    dense, none = run_distributed(_train, 1, [])[0]
    assert all(math.isfinite(v) for v in dense) and not none
    sparse, kl = run_distributed(_train, 1, DSA)[0]
    assert sparse != dense and all(math.isfinite(v) for v in sparse) and sorted(kl) == [1, 2, 3, 4] and all(v > 0 for v in kl.values())
    absorbed, kl_a = run_distributed(_train, 1, DSA + ["--use-dsa-absorb"])[0]
    # rounding differences can flip a top-k choice later on, so the trajectories are compared over the first steps
    assert all(abs(a - b) < 1e-4 for a, b in zip(sparse[:3], absorbed[:3])), (sparse, absorbed)
    # heads split over two ranks, sequence parallel: same model, same trajectory
    tp = run_distributed(_train, 2, DSA + ["--tensor-model-parallel-size", "2", "--sequence-parallel"])
    assert all(abs(a - b) < 1e-4 for a, b in zip(sparse[:3], tp[0][0][:3])), (sparse, tp[0][0])
    assert all(abs(kl[k] - tp[0][1][k]) < 0.05 * kl[k] for k in kl), (kl, tp[0][1])
