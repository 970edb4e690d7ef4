"""Context-parallel attention on CPU/gloo against full-sequence attention on one rank (out, dq, dk, dv)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


def _full(seed, s, b, nq, nkv, d):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(s, b, nq, d, generator=g)
    k = torch.randn(s, b, nkv, d, generator=g)
    v = torch.randn(s, b, nkv, d, generator=g)
    w = torch.randn(s, b, nq, d, generator=g)
    return q, k, v, w


def _run(rank, world, algo, nq, nkv, causal, extra):
    import torch.distributed as dist
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.context_parallel import dispatch_context_parallel_attention
    from mindspeed_b200.parallel.context_parallel.batch_utils import slice_for_cp
    dist.init_process_group("gloo", rank=rank, world_size=world)
    kw = dict(context_parallel_size=world, use_cp_send_recv_overlap=extra.get("overlap", False))
    if algo == "hybrid_cp_algo":
        kw["ulysses_degree_in_cp"] = 2
    ps.initialize_model_parallel(**kw)
    cfg = TransformerConfig(num_layers=1, hidden_size=nq * 16, num_attention_heads=nq, num_query_groups=nkv,
                            context_parallel_size=world, use_cpu_initialization=True, optimization_level=0)
    cfg.context_parallel_algo = algo
    cfg.context_parallel_kv_cache_policy = extra.get("cache")
    cfg.context_parallel_cache_interval = 0
    cfg.use_ulysses_allgather_kv = bool(extra.get("allgather_kv", False))
    cfg.hamilton_path_num = extra.get("paths", 0)
    cfg.cp_window_size = extra.get("window", 1)
    s, b, d = 32 * world, 2, 16
    q, k, v, w = _full(3, s, b, nq, nkv, d)
    if extra.get("dv"):
        v, w = v[..., :extra["dv"]].contiguous(), w[..., :extra["dv"]].contiguous()
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal=causal)
    (ref * w).sum().backward()
    sl = lambda t: slice_for_cp(t, 0, algo).clone()
    ql, kl, vl = (sl(t).requires_grad_(True) for t in (q, k, v))
    out = dispatch_context_parallel_attention(ql, kl, vl, cfg, causal=causal)
    (out * sl(w)).sum().backward()
    res = {}
    res["out"] = (out.detach() - sl(ref.detach())).abs().max().item()
    res["dq"] = (ql.grad - sl(qf.grad)).abs().max().item()
    res["dk"] = (kl.grad - sl(kf.grad)).abs().max().item()
    res["dv"] = (vl.grad - sl(vf.grad)).abs().max().item()
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return res


@pytest.mark.parametrize("algo,world,nq,nkv,causal,extra", [
    ("megatron_cp_algo", 2, 4, 2, True, {}),
    ("megatron_cp_algo", 4, 4, 4, True, {"overlap": True, "cache": "full"}),
    ("ulysses_cp_algo", 2, 4, 2, True, {}),
    ("ulysses_cp_algo", 4, 4, 2, True, {}),
    ("ulysses_cp_algo", 4, 4, 2, True, {"allgather_kv": True}),       # fewer KV heads than ranks: K/V gathered along the sequence
    ("ulysses_cp_algo", 2, 4, 1, True, {"allgather_kv": True}),
    # double ring: hops inside windows of 2, then across windows; gradients return straight to the block's origin
    ("megatron_cp_algo", 4, 4, 2, True, {"window": 2}),
    ("megatron_cp_algo", 6, 2, 2, True, {"window": 3}),
    ("megatron_cp_algo", 4, 4, 4, False, {"window": 2}),
    # K and V with different head dimensions (multi-latent attention) travel as one concatenated message
    ("megatron_cp_algo", 4, 4, 4, True, {"dv": 8}),
    ("megatron_cp_algo", 4, 4, 4, True, {"dv": 8, "window": 2}),
    ("kvallgather_cp_algo", 2, 4, 2, True, {}),
    ("hybrid_cp_algo", 4, 4, 4, True, {}),
    # Hamilton: the KV block split over edge-disjoint cycles (strides coprime to the group size), full attention
    ("hamilton_cp_algo", 4, 4, 2, False, {}),                  # 4 ranks: strides 1 and 3
    ("hamilton_cp_algo", 5, 4, 4, False, {"paths": 4}),        # 5 ranks: strides 1, 2, 3, 4
    ("hamilton_cp_algo", 3, 2, 1, False, {"paths": 1}),        # one path = a plain ring
])
def test_cp_attention_matches_full(algo, world, nq, nkv, causal, extra):
    for r in run_distributed(_run, world, algo, nq, nkv, causal, extra):
        for key, err in r.items():
            assert err < 2e-4, (algo, key, err, r)


def _run_adaptive(rank, world):
    import torch.distributed as dist
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.context_parallel.adaptive import adaptive_attention
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(context_parallel_size=world)
    s, b, n, d = 16 * world, 1, 2, 8
    q, k, v, w = _full(5, s, b, n, n, d)
    g = torch.Generator().manual_seed(11)
    # band + a few global tokens, never fully masked rows
    idx = torch.arange(s)
    mask = ((idx.view(-1, 1) - idx.view(1, -1)).abs() > 12) & (idx.view(1, -1) > 1)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal=False, mask=mask.view(1, 1, s, s))
    (ref * w).sum().backward()
    per = s // world
    sl = lambda t: t[rank * per:(rank + 1) * per].clone()
    ql, kl, vl = (sl(t).requires_grad_(True) for t in (q, k, v))
    out = adaptive_attention(ql, kl, vl, None, mask)
    (out * sl(w)).sum().backward()
    # the same mask handed over block by block (--adaptive-cp-manually-set-mask-list): same result, schedule from the list
    from mindspeed_b200.parallel.context_parallel import adaptive as AD
    import types
    blocks = [[None if bool(mask[i * per:(i + 1) * per, j * per:(j + 1) * per].all()) else
               mask[i * per:(i + 1) * per, j * per:(j + 1) * per].clone() for j in range(world)] for i in range(world)]
    AD.set_block_mask_list(blocks)
    cfg = types.SimpleNamespace(adaptive_cp_manually_set_mask_list=True, adaptive_cp_dynamic_attn_mask=True, adaptive_cp_comm_limit=1)
    q2, k2, v2 = (sl(t).requires_grad_(True) for t in (q, k, v))
    out2 = adaptive_attention(q2, k2, v2, cfg, None)
    assert (out2.detach() - out.detach()).abs().max().item() < 1e-6
    n_cached = len(AD._SCHEDULE_CACHE)
    adaptive_attention(sl(q), sl(k), sl(v), None, mask)           # static mask: the schedule is reused
    assert len(AD._SCHEDULE_CACHE) == n_cached
    res = {"out": (out.detach() - sl(ref.detach())).abs().max().item(), "dq": (ql.grad - sl(qf.grad)).abs().max().item(),
           "dk": (kl.grad - sl(kf.grad)).abs().max().item(), "dv": (vl.grad - sl(vf.grad)).abs().max().item()}
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return res


def test_adaptive_cp_matches_masked_attention():
    for r in run_distributed(_run_adaptive, 4):
        for key, err in r.items():
            assert err < 2e-4, (key, err, r)


def test_adaptive_cp_host_algorithms():
    from mindspeed_b200.parallel.context_parallel.adaptive import coarsen_mask, schedule_rounds, search_kmeans
    S, blk = 64, 8
    idx = torch.arange(S)
    visible = (idx.view(-1, 1) - idx.view(1, -1)).abs() < 10
    c = coarsen_mask(visible, blk)
    ref = visible.view(8, blk, 8, blk).any(dim=3).any(dim=1)
    assert torch.equal(c.bool(), ref)
    rounds, ro = schedule_rounds(c, comm_limit=1)
    need = c.bool() & ~torch.eye(8, dtype=torch.bool)
    assert ((ro >= 0) == need).all()
    for rd in range(rounds):                      # per round: each rank receives <= 1 and sends <= 1
        m = ro == rd
        assert m.sum(1).max() <= 1 and m.sum(0).max() <= 1
    # two interleaved document families: k-means should separate them
    fam = torch.arange(8) % 2
    c2 = (fam.view(-1, 1) == fam.view(1, -1)).to(torch.uint8)
    order = search_kmeans(c2, 2)
    assert sorted(order) == list(range(8))
    assert len({int(fam[i]) for i in order[:4]}) == 1 and len({int(fam[i]) for i in order[4:]}) == 1


def test_hamilton_cycles_are_hamiltonian_and_edge_disjoint():
    from mindspeed_b200.parallel.context_parallel.hamilton import hamilton_strides, max_paths
    for n in (2, 3, 4, 5, 8, 12):
        strides = hamilton_strides(n, max_paths(n))
        edges = set()
        for s in strides:
            seen, r = set(), 0
            for _ in range(n):
                seen.add(r)
                e = (r, (r + s) % n)
                assert e not in edges
                edges.add(e)
                r = (r + s) % n
            assert len(seen) == n and r == 0        # visits every rank once and closes
    with pytest.raises(ValueError):
        hamilton_strides(8, 5)                      # 8 ranks have 4 such cycles


def test_double_ring_schedule_is_consistent():
    from mindspeed_b200.parallel.context_parallel.ring import ring_schedule
    for cp, w in ((4, 1), (4, 2), (8, 4), (8, 2), (6, 3)):
        sch = [ring_schedule(cp, r, w) for r in range(cp)]
        for r in range(cp):
            src, send_to, recv_from, home = sch[r]
            assert sorted(src) == list(range(cp)) and src[0] == r          # every block once, the local one first
            for i in range(cp - 1):
                assert sch[send_to[i]][2][i] == r                          # my receiver expects me
                assert sch[recv_from[i]][0][i] == src[i + 1]               # and I get the block my sender was working on
                if w > 1:
                    same_window = send_to[i] // w == r // w
                    assert same_window == (i % w != w - 1)                 # w - 1 inner hops, then one outer hop
            assert sch[home][0][cp - 1] == r                               # my block's gradient comes home from its last holder
    with pytest.raises(ValueError):
        ring_schedule(6, 0, 4)


def _unaligned_ulysses(rank, world, total):
    import torch.distributed as dist
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.parallel.context_parallel import ulysses as U
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    b, n, d = 2, 4, 8
    q, k, v = (torch.randn(total, b, n, d, generator=g) for _ in range(3))
    lens = U.split_lengths(total, world)
    lo = sum(lens[:rank])
    sl = slice(lo, lo + lens[rank])
    ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
    out = U.ulysses_attention(ql, kl, vl, None, dist.group.WORLD, causal=True,
                              inner=lambda a, b_, c: attention_ref(a, b_, c, causal=True),
                              gather_size_calculator=U.DynamicGatherSizeCalculator(), attention_mask=total)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal=True)
    w = torch.randn(total, b, n, d, generator=g)
    (out * w[sl]).sum().backward()
    (ref * w).sum().backward()
    # gradients of K / V on this rank's slice collect contributions of every rank's queries through the all-to-alls
    ok = torch.allclose(out, ref[sl], atol=1e-5) and torch.allclose(ql.grad, qf.grad[sl], atol=1e-5) \
        and torch.allclose(kl.grad, kf.grad[sl], atol=1e-5) and torch.allclose(vl.grad, vf.grad[sl], atol=1e-5)
    dist.destroy_process_group()
    return ok, lens


def test_ulysses_with_a_sequence_length_the_group_does_not_divide():
    from mindspeed_b200.parallel.context_parallel.ulysses import DefaultGatherSizeCalculator, DynamicGatherSizeCalculator, split_lengths
    assert split_lengths(10, 4) == [3, 3, 2, 2] and split_lengths(8, 4) == [2, 2, 2, 2]
    assert DefaultGatherSizeCalculator().calculate() is None
    assert DynamicGatherSizeCalculator().calculate(attention_mask=torch.zeros(1, 1, 7, 7)) == 7
    res = run_distributed(_unaligned_ulysses, 2, 13)
    assert all(ok for ok, _ in res) and res[0][1] == [7, 6]
    res = run_distributed(_unaligned_ulysses, 4, 10)
    assert all(ok for ok, _ in res)


def _unaligned_ring(rank, world, lens):
    import torch.distributed as dist
    from mindspeed_b200.ops.attention import attention_ref
    from mindspeed_b200.parallel.context_parallel.ring import ring_attention
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    total, b, n, d = sum(lens), 2, 2, 8
    q, k = torch.randn(total, b, n, d, generator=g), torch.randn(total, b, n, d, generator=g)
    v = torch.randn(total, b, n, d, generator=g)
    lo = sum(lens[:rank])
    sl = slice(lo, lo + lens[rank])
    ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
    out = ring_attention(ql, kl, vl, None, causal=False, group=dist.group.WORLD, ranks=list(range(world)), shapes=lens)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal=False)
    w = torch.randn(total, b, n, d, generator=g)
    (out * w[sl]).sum().backward()
    (ref * w).sum().backward()
    ok = torch.allclose(out, ref[sl], atol=1e-5) and torch.allclose(ql.grad, qf.grad[sl], atol=1e-5) \
        and torch.allclose(kl.grad, kf.grad[sl], atol=1e-5) and torch.allclose(vl.grad, vf.grad[sl], atol=1e-5)
    dist.destroy_process_group()
    return ok


@pytest.mark.parametrize("lens", [[5, 3], [5, 3, 4], [2, 6, 1, 4]])
def test_ring_attention_over_slices_of_different_lengths(lens):
    assert all(run_distributed(_unaligned_ring, len(lens), lens))
