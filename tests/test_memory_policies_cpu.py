"""Smart swap (profile -> policy -> execute), adaptive recompute (profile -> knapsack -> apply), auto pipeline split."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from mindspeed_b200.memory import adaptive_recompute as AR
from mindspeed_b200.memory import auto_pipeline as AP
from mindspeed_b200.memory import smart_swap as SS


class Blk(nn.Module):
    def __init__(self, h):
        super().__init__()
        self.a, self.b = nn.Linear(h, 4 * h), nn.Linear(4 * h, h)

    def forward(self, x):
        return x + self.b(torch.tanh(self.a(x)))


def _net(n=4, h=64):
    torch.manual_seed(0)
    return nn.Sequential(*[Blk(h) for _ in range(n)])


def test_smart_swap_phases_and_numerics():
    net = _net()
    x = torch.randn(256, 64, requires_grad=True)
    ref = net(x).pow(2).sum()
    ref.backward()
    gref = [p.grad.clone() for p in net.parameters()]
    net.zero_grad()
    mgr = SS.SmartSwapManager(budget_bytes=300_000, warmup_steps=1, min_bytes=1 << 12, op_time=1e-3, d2h_gbs=1.0, h2d_gbs=1.0)
    with mgr.step_context():
        loss = net(x).pow(2).sum()
    loss.backward()
    net.zero_grad()
    prof = mgr.profiler
    assert prof.lives and all(l.use_op >= 0 for l in prof.lives)
    gen = SS.PolicyGenerator(prof.lives, prof.num_forward_ops, prof.num_backward_ops, op_time=1e-3, d2h_gbs=1.0, h2d_gbs=1.0)
    base_peak = max(gen.timeline())
    mgr.end_step()
    assert mgr.phase == "stable" and mgr.policy.swap_keys
    assert mgr.policy.expected_peak < base_peak
    # tensors alive at the peak and with long idle time are preferred: the earliest big saves
    first = min(prof.lives, key=lambda l: l.save_op)
    assert first.key in mgr.policy.swap_keys
    with mgr.step_context() as ex:
        loss = net(x).pow(2).sum()
    loss.backward()
    assert ex.n_swapped == len(mgr.policy.swap_keys) and ex.bytes_swapped > 0
    assert torch.allclose(loss, ref)
    for p, g in zip(net.parameters(), gref):
        assert torch.allclose(p.grad, g, atol=1e-6)


def test_policy_respects_copy_bandwidth():
    lives = [SS.TensorLife(0, 100 << 20, 0, 99), SS.TensorLife(1, 100 << 20, 48, 51)]
    gen = SS.PolicyGenerator(lives, 50, 100, op_time=1e-3, d2h_gbs=10.0, h2d_gbs=10.0)
    pol = gen.generate(budget_bytes=150 << 20)
    assert pol.swap_keys == [0]          # tensor 1 lives too briefly around the peak for its copies to hide


def test_knapsack_prefers_cheap_bytes():
    P = AR.ModuleProfile
    profs = [P("l0", 3.0, 100 << 20, 10 << 20, 1), P("l0.attn", 1.0, 70 << 20, 10 << 20, 1, "l0"), P("l0.mlp", 1.5, 20 << 20, 10 << 20, 1, "l0"),
             P("l1", 3.0, 100 << 20, 10 << 20, 1), P("l1.attn", 1.0, 70 << 20, 10 << 20, 1, "l1"), P("l1.mlp", 1.5, 20 << 20, 10 << 20, 1, "l1")]
    assert AR.solve_recompute(profs, 0) == []
    assert sorted(AR.solve_recompute(profs, 50 << 20)) in (["l0.attn"], ["l1.attn"])
    assert sorted(AR.solve_recompute(profs, 120 << 20)) == ["l0.attn", "l1.attn"]
    assert sorted(AR.solve_recompute(profs, 170 << 20)) == ["l0", "l1"] or len(AR.solve_recompute(profs, 170 << 20)) >= 2
    assert sorted(AR.solve_recompute(profs, 10_000 << 20)) == ["l0", "l1"]


def test_adaptive_recompute_end_to_end():
    net = _net(3)
    x = torch.randn(128, 64, requires_grad=True)
    names = ["0", "1", "2"]
    ar = AR.AdaptiveRecompute(net, candidates=names, profiling_steps=1, device_budget_bytes=200_000)
    with ar.step_context():
        loss = net(x).pow(2).sum()
    loss.backward()
    gref = [p.grad.clone() for p in net.parameters()]
    net.zero_grad()
    ar.end_step(static_bytes=0)
    assert all(ar.profiles[n].saved_bytes > 0 and ar.profiles[n].forward_time > 0 for n in names)
    assert ar.chosen and all(isinstance(getattr(net, n), AR._Ckpt) for n in ar.chosen)
    with ar.step_context():
        loss2 = net(x).pow(2).sum()
    loss2.backward()
    assert torch.allclose(loss, loss2)
    got = [p.grad for p in net.parameters()]
    assert all(torch.allclose(a, b, atol=1e-6) for a, b in zip(got, gref))


def test_adaptive_recompute_parks_activations_on_the_host_while_profiling():
    """``swap_while_profiling``: during the profiling steps saved tensors go through the host-offload hooks (here a stand-in
    that wraps them, as CPU tensors are passed through by the real one); after the decision the hooks are gone."""
    net = _net(3)
    x = torch.randn(128, 64, requires_grad=True)
    ar = AR.AdaptiveRecompute(net, candidates=["0", "1", "2"], profiling_steps=1, device_budget_bytes=200_000,
                              swap_while_profiling=True, swap_min_bytes=1024)
    assert ar.swap is not None and ar.swap.min_bytes == 1024
    parked = {"out": 0, "back": 0}

    class Box:
        def __init__(self, t):
            self.t = t

    class FakeSwap:
        def _pack(self, t):
            if t.numel() * t.element_size() < 1024:
                return t
            parked["out"] += 1
            return Box(t.clone())

        def _unpack(self, o):
            if isinstance(o, Box):
                parked["back"] += 1
                return o.t
            return o
    ar.swap = FakeSwap()
    with ar.step_context():
        loss = net(x).pow(2).sum()
    loss.backward()
    gref = [p.grad.clone() for p in net.parameters()]
    net.zero_grad()
    assert parked["out"] > 0 and parked["back"] == parked["out"] and ar.swapped_bytes > 0
    ar.end_step(static_bytes=0)
    assert ar.chosen and all(ar.profiles[n].saved_bytes > 0 for n in ("0", "1", "2"))      # byte counts unaffected by the swap
    n_out = parked["out"]
    with ar.step_context():
        loss2 = net(x).pow(2).sum()
    loss2.backward()
    assert parked["out"] == n_out                                                           # no swap after profiling
    assert torch.allclose(loss, loss2)
    assert all(torch.allclose(a.grad, b, atol=1e-6) for a, b in zip(net.parameters(), gref))


def test_adaptive_memory_chooses_between_recompute_and_host_swap():
    from mindspeed_b200.memory import adaptive_memory as AM
    MP = AR.ModuleProfile
    MB = 1 << 20
    layers = [MP(f"l{i}", forward_time=0.010, saved_bytes=400 * MB, input_bytes=40 * MB) for i in range(4)]
    fast, slow = AM.HostLink(bytes_per_s=60e9, latency_s=2e-5), AM.HostLink(bytes_per_s=2e9, latency_s=2e-5)
    # a fast link hides the copies behind the layer's own compute: swapping is (nearly) free and frees more than recompute
    pol = AM.solve_memory_policy(layers, 700 * MB, fast)
    assert sorted(pol.values()) == ["swap", "swap"]
    # a slow link exposes 2 * (0.2 s - 0.01 s) per layer: one more forward (10 ms) is cheaper
    pol = AM.solve_memory_policy(layers, 700 * MB, slow)
    assert sorted(pol.values()) == ["recompute", "recompute"]
    assert AM.solve_memory_policy(layers, 700 * MB, fast, allow_swap=False) == pol
    assert AM.solve_memory_policy(layers, 0, fast) == {}
    # activations of several micro-batches in flight on a pipeline stage: one layer's action frees in_flight times as much
    assert len(AM.solve_memory_policy(layers, 700 * MB, fast, in_flight=2)) == 1
    # children are an alternative to the whole layer: only the attention part is cheap to swap here
    tree = [MP("l0", 0.010, 400 * MB, 40 * MB), MP("l0.attn", 0.008, 100 * MB, 40 * MB, parent="l0"),
            MP("l0.mlp", 0.002, 300 * MB, 40 * MB, parent="l0")]
    mid = AM.HostLink(bytes_per_s=20e9, latency_s=2e-5)            # attn: 5 ms copy < 8 ms compute; mlp: 15 ms copy > 2 ms
    assert AM.solve_memory_policy(tree, 90 * MB, mid) == {"l0.attn": "swap"}
    assert AM.solve_memory_policy(tree, 250 * MB, mid) == {"l0.mlp": "recompute"}
    # unreachable target: everything that frees the most
    assert set(AM.solve_memory_policy(layers, 10_000 * MB, slow).values()) == {"swap"}


def test_adaptive_memory_end_to_end_applies_both_wrappers():
    from mindspeed_b200.memory import adaptive_memory as AM
    net = _net(3)
    x = torch.randn(128, 64, requires_grad=True)
    parked = {"n": 0}

    class Ctx:
        def __enter__(self):
            parked["n"] += 1

        def __exit__(self, *a):
            return False
    # layer "0" gets a huge compute time through a fast fake link -> swap; the link is slow for the rest -> recompute
    am = AM.AdaptiveMemory(net, candidates=["0", "1", "2"], profiling_steps=1, device_budget_bytes=1, allow_swap=True,
                           link=AM.HostLink(bytes_per_s=1e6, latency_s=0.0), swap_context=Ctx, granularity=1024)
    with am.step_context():
        loss = net(x).pow(2).sum()
    loss.backward()
    gref = [p.grad.clone() for p in net.parameters()]
    net.zero_grad()
    am.profiles["0"].forward_time = 10.0                           # its copies hide completely
    pr = am.profiles
    total = sum(p.saved_bytes for p in pr.values())
    # what must go: all of layer 0 (only a swap frees that much) and the recomputable part of the other two
    am.budget = total - (pr["0"].saved_bytes + sum(pr[n].saved_bytes - pr[n].input_bytes for n in ("1", "2"))) + 1024
    am.end_step(static_bytes=0)
    assert am.policy["0"] == "swap" and isinstance(getattr(net, "0"), AM._Swap)
    assert all(am.policy[n] == "recompute" and isinstance(getattr(net, n), AR._Ckpt) for n in ("1", "2"))
    with am.step_context():
        loss2 = net(x).pow(2).sum()
    loss2.backward()
    assert parked["n"] == 1 and torch.allclose(loss, loss2)
    assert all(torch.allclose(a.grad, b, atol=1e-6) for a, b in zip(net.parameters(), gref))


def test_auto_pipeline_balances_time_under_memory():
    LP = AP.LayerProfile
    layers = [LP(1.0, 2.0, 100, 10, 50) for _ in range(8)]
    plan = AP.solve_pipeline(layers, pp=4, n_mb=8, budget_bytes=10_000)
    assert plan.feasible and plan.layers_per_stage == [2, 2, 2, 2] and plan.recompute_per_stage == [0, 0, 0, 0]
    # a tight budget: early stages hold more micro-batches in flight, so they must recompute (or take fewer layers)
    tight = AP.solve_pipeline(layers, pp=4, n_mb=8, budget_bytes=2 * 50 + 4 * 120)
    assert tight.feasible and tight.recompute_per_stage[0] >= tight.recompute_per_stage[-1]
    assert all(b <= 2 * 50 + 4 * 120 for b in tight.stage_bytes)
    # heterogeneous layers: the split follows time, not count
    layers2 = [LP(1.0, 2.0, 10, 1, 5)] * 4 + [LP(3.0, 6.0, 10, 1, 5)] * 4
    p2 = AP.solve_pipeline(layers2, pp=2, n_mb=4, budget_bytes=10_000)
    assert p2.layers_per_stage == [5, 3]
    none = AP.solve_pipeline(layers, pp=4, n_mb=8, budget_bytes=10)
    assert not none.feasible
    mbs, plan = AP.search_micro_batch(lambda m: [LP(1.0 * m ** 0.9, 2.0 * m ** 0.9, 100 * m, 10 * m, 50) for _ in range(8)],
                                      [1, 2, 4], global_batch=32, dp=1, pp=4, budget_bytes=3000)
    assert mbs in (1, 2, 4) and plan.feasible


def _train_compress(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.memory import compress_activation as CA
    from mindspeed_b200.training import pretrain
    CA.MIN_NUMEL = 256                       # the test model's activations are tiny
    CA.reset_stats()
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + list(extra))
    return [h["lm loss"] for h in hist], dict(CA.CompressSavedActivations.stats)


def test_compress_activation_is_lossless_and_smaller():
    """``--compress-activation`` / ``--compress-dense``: identical losses (the codec is bit-exact) and fewer stored bytes."""
    from dist_utils import run_distributed
    ref, st0 = run_distributed(_train_compress, 1, [])[0]
    assert st0["tensors"] == 0
    for extra in (["--compress-activation", "1,3-4"], ["--compress-activation", "0"], ["--compress-dense", "level1"],
                  ["--compress-dense", "level0"]):
        got, st = run_distributed(_train_compress, 1, extra)[0]
        assert got == ref, (extra, ref, got)
        assert st["tensors"] > 0 and st["stored"] < 0.95 * st["raw"], (extra, st)
    # Adam moments held encoded between steps: same trajectory, with and without the distributed optimizer
    got, _ = run_distributed(_train_compress, 1, ["--compress-optimizer"])[0]
    assert got == ref, (ref, got)
    ref2 = run_distributed(_train_compress, 2, ["--use-distributed-optimizer"])[0][0]
    got2 = run_distributed(_train_compress, 2, ["--use-distributed-optimizer", "--compress-optimizer"])[0][0]
    assert got2 == ref2, (ref2, got2)


def test_compress_activation_layer_spec():
    from mindspeed_b200.memory.compress_activation import parse_layers
    assert parse_layers("0", 4) == [1, 2, 3, 4]
    assert parse_layers("1,3-4", 6) == [1, 3, 4]
    assert parse_layers("", 4) == []
    with pytest.raises(ValueError):
        parse_layers("5", 4)


def test_automated_pipeline_gives_the_output_stage_fewer_layers():
    import types
    from mindspeed_b200.memory.auto_pipeline import plan_from_args
    a = types.SimpleNamespace(micro_batch_size=1, tensor_model_parallel_size=1, context_parallel_size=1, seq_length=8192,
                              hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=14336,
                              swiglu=True, num_experts=None, moe_router_topk=1, expert_model_parallel_size=1, num_layers=32,
                              padded_vocab_size=128256, sequence_parallel=False, pipeline_model_parallel_size=4, world_size=8,
                              global_batch_size=64, use_distributed_optimizer=True, adaptive_recompute_device_size=-1)
    mbs, plan = plan_from_args(a)
    assert mbs == 1 and plan.feasible and sum(plan.layers_per_stage) == 32
    assert plan.layers_per_stage[-1] < max(plan.layers_per_stage)           # the 128k-vocabulary head costs about two layers
    assert max(plan.stage_times) / min(plan.stage_times) < 1.2
    # a tight budget forces recompute on the early stages, which hold the most micro-batches in flight
    a.adaptive_recompute_device_size = 40 * 1024
    _, tight = plan_from_args(a)
    assert tight.feasible and tight.recompute_per_stage[0] >= tight.recompute_per_stage[-1] and sum(tight.recompute_per_stage) > 0


def test_quant_grads_uses_16_bit_gradient_buffers():
    """``--quant-grads``: gradient accumulation and data-parallel reduction in fp16 buffers; the trajectory stays close."""
    from dist_utils import run_distributed
    ref = run_distributed(_train_compress, 2, ["--use-distributed-optimizer"])[0][0]
    got = run_distributed(_train_compress, 2, ["--use-distributed-optimizer", "--quant-grads"])[0][0]
    assert got != ref                                   # the buffers really are 16-bit
    for a, b in zip(ref, got):
        assert abs(a - b) < 5e-3 * max(1.0, abs(a)), (ref, got)
