"""Pipeline schedules: plan validity for every schedule, and gloo multi-rank numerics against no pipelining."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402


@pytest.mark.parametrize("name,vpp", [("1f1b", None), ("interleaved", 2), ("interleaved", 4), ("nanopipe", 2), ("dualpipev", None),
                                      ("dualpipev_greedy", None), ("dualpipe", None), ("chimera", None)])
@pytest.mark.parametrize("pp", [2, 4, 8])
def test_plans_are_valid_and_matched(name, vpp, pp):
    from mindspeed_b200.parallel.pipeline.plan import build_plan, validate
    for n in (2 * pp, 4 * pp):
        plan = build_plan(name, pp, n, vpp=vpp)
        validate(plan)
        # every message is received in the slot it is sent, and its consumer runs no earlier than that slot
        for m in plan.messages:
            ops = plan.table[m.dst][m.slot:]
            kind = "F" if m.kind == "act" else "B"
            assert any(o.kind == kind and o.chunk == m.dst_chunk and o.mb == m.mb for slot in ops for o in slot), m
        for (r, t), sends in plan.sends.items():
            for m in sends:
                assert m in plan.recvs[(m.dst, t)]


@pytest.mark.parametrize("mode", ["bubble", "advance"])
def test_recompute_ops_fill_bubbles(mode):
    from mindspeed_b200.parallel.pipeline.plan import build_plan, validate
    pp, n = 4, 8
    base = build_plan("1f1b", pp, n)
    plan = build_plan("1f1b", pp, n, recompute=mode)
    validate(plan)
    for r in range(pp):
        ops = [o for slot in plan.table[r] for o in slot]
        rs = {(o.chunk, o.mb) for o in ops if o.kind == "R"}
        # the last stage runs B right after F: it never recomputes; earlier stages recompute the micro-batches in flight
        assert (len(rs) == 0) == (r == pp - 1)
        for (c, mb) in rs:
            i_f = ops.index(next(o for o in ops if o.kind == "F" and (o.chunk, o.mb) == (c, mb)))
            i_r = ops.index(next(o for o in ops if o.kind == "R" and (o.chunk, o.mb) == (c, mb)))
            i_b = ops.index(next(o for o in ops if o.kind == "B" and (o.chunk, o.mb) == (c, mb)))
            assert i_f < i_r < i_b
    # timed simulation: scheduler-placed recompute must beat recompute inside every backward (B = 2 + 1), because it
    # skips the forwards that are followed directly by their backward and runs the rest while waiting for gradients
    from mindspeed_b200.parallel.pipeline.plan import insert_recompute, order_1f1b, placement_1f1b, simulate_orders
    pl, orders = placement_1f1b(pp), order_1f1b(pp, n)
    t_none, _ = simulate_orders(pl, orders, {"F": 1, "B": 2, "W": 0})
    t_naive, _ = simulate_orders(pl, orders, {"F": 1, "B": 3, "W": 0})
    t_ri, _ = simulate_orders(pl, insert_recompute(orders, mode), {"F": 1, "B": 2, "W": 0, "R": 1})
    assert t_none <= t_ri < t_naive, (t_none, t_ri, t_naive)


def test_nanopipe_defers_the_first_weight_gradients_of_each_rank_and_shortens_the_step():
    from mindspeed_b200.parallel.pipeline.plan import order_interleaved, placement_interleaved, simulate_orders
    pp, v, n = 4, 2, 8
    plain, nano = order_interleaved(pp, v, n), order_interleaved(pp, v, n, nano=True)
    for r in range(pp):
        ops = nano[r]
        assert [o for o in ops if o.kind != "W"] == plain[r]                   # same forward / backward order
        bs = [o for o in ops if o.kind == "B"]
        ws = [o for o in ops if o.kind == "W"]
        assert sorted((o.chunk, o.mb) for o in bs) == sorted((o.chunk, o.mb) for o in ws)
        last_b = max(i for i, o in enumerate(ops) if o.kind == "B")
        late = [o for o in ops[last_b + 1:] if o.kind == "W"]
        assert len(late) == 2 * r + 1                                            # the last backward's own, then the deferred ones
        assert [(o.chunk, o.mb) for o in late[1:]] == [(o.chunk, o.mb) for o in bs[:2 * r]]
    # with backward split into equal input- and weight-gradient parts the deferral shortens the step
    cost = {"F": 1, "B": 1, "W": 1}
    pl = placement_interleaved(pp, v)
    both = [[x for o in ops for x in ((o, type(o)("W", o.chunk, o.mb)) if o.kind == "B" else (o,))] for ops in plain]
    t_plain, _ = simulate_orders(pl, both, cost)
    t_nano, _ = simulate_orders(pl, nano, cost)
    assert t_nano < t_plain, (t_nano, t_plain)


def test_1f1b_bubble_matches_theory():
    from mindspeed_b200.parallel.pipeline.plan import order_1f1b, placement_1f1b, simulate_orders, greedy_orders, placement_v
    for pp, n in ((4, 8), (8, 32)):
        _, bub = simulate_orders(placement_1f1b(pp), order_1f1b(pp, n), {"F": 1, "B": 2, "W": 0})
        assert abs(bub - (pp - 1) / (n + pp - 1)) < 1e-6
        # the V schedule with split weight gradients must beat 1F1B's bubble
        _, bub_v = simulate_orders(placement_v(pp), greedy_orders(placement_v(pp), n, True), {"F": 1, "B": 1, "W": 1})
        assert bub_v < 0.5 * bub


BASE = ["--num-layers", "4", "--hidden-size", "64", "--num-attention-heads", "4", "--ffn-hidden-size", "128", "--seq-length", "32",
        "--max-position-embeddings", "32", "--micro-batch-size", "1", "--global-batch-size", "8", "--vocab-size", "128",
        "--make-vocab-size-divisible-by", "1", "--train-iters", "3", "--lr", "1e-3", "--lr-decay-style", "constant",
        "--hidden-dropout", "0", "--attention-dropout", "0", "--seed", "1234", "--distributed-backend", "gloo",
        "--optimization-level", "0", "--use-cpu-initialization", "--weight-decay", "0.0", "--clip-grad", "0.0",
        "--untie-embeddings-and-output-weights", "--swiglu", "--normalization", "RMSNorm", "--position-embedding-type", "rope",
        "--disable-bias-linear", "--no-gradient-accumulation-fusion"]


def _canonical_init(model):
    """Give every parameter a value that depends only on its global name, so any pipeline layout holds the same model."""
    import hashlib
    for chunk in model:
        inner = chunk.module if hasattr(chunk, "module") else chunk
        for name, p in inner.named_parameters():
            parts = name.split(".")
            if "layers" in parts:
                i = parts.index("layers")
                layer = inner.decoder.layers[int(parts[i + 1])]
                parts[i + 1] = str(layer.layer_number)
            key = ".".join(parts)
            seed = int(hashlib.sha256(key.encode()).hexdigest()[:8], 16)
            g = torch.Generator().manual_seed(seed)
            with torch.no_grad():
                if p.dim() == 1:
                    p.copy_(1.0 + 0.01 * torch.randn(p.shape, generator=g))
                else:
                    p.copy_(0.05 * torch.randn(p.shape, generator=g))


def _train(rank, world, extra, bidirectional):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.pipeline.executor import current_microbatch
    from mindspeed_b200.training import get_args, initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import SyntheticGPTDataset
    args = initialize_megatron(args_list=BASE + list(extra))
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    _canonical_init(model)
    if bidirectional:
        from mindspeed_b200.parallel.pipeline.chimera import sync_replica_params
        sync_replica_params(model)
    opt.reload_model_params()
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
    nmb = args.global_batch_size // args.micro_batch_size
    state = {"step": 0}

    class It:
        """Data keyed by (step, pipeline, micro-batch) so every layout sees the same global batch."""
        def __iter__(self):
            return self

        def __next__(self):
            cur = current_microbatch()
            mb = cur["mb"] + (cur["pipe"] * (nmb // 2) if bidirectional else 0)
            item = ds[state["step"] * nmb + mb]
            return {k: v.unsqueeze(0) for k, v in item.items()}

    class Plain:
        def __init__(self):
            self.i = 0

        def __iter__(self):
            return self

        def __next__(self):
            item = ds[self.i]
            self.i += 1
            return {k: v.unsqueeze(0) for k, v in item.items()}

    it = It() if ps.get_pipeline_model_parallel_world_size() > 1 else Plain()
    out = []
    for _ in range(3):
        ld, *_ = train_step(pg.forward_step, [it] * len(model) if len(model) > 1 else it, model, opt, sched)
        state["step"] += 1
        out.append(float(ld["lm loss"]) if "lm loss" in ld else None)
    return out


_REF = {}


def _reference_losses(model_flags):
    """The one-rank run every pipeline layout is compared with (computed once per model shape)."""
    if model_flags not in _REF:
        _REF[model_flags] = run_distributed(_train, 1, list(model_flags), False)[0]
    return _REF[model_flags]


@pytest.mark.parametrize("world,extra,bidir", [
    (2, ["--pipeline-model-parallel-size", "2"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipev"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--recompute-in-bubble"], False),
    # layers per stage chosen from the model shape (the stage with the output layer gets fewer transformer layers)
    (2, ["--pipeline-model-parallel-size", "2", "--automated-pipeline", "--vocab-size", "2048", "--num-layers", "5"], False),
    # a stored automated-pipeline policy: layers per rank, and per rank how many layers recompute their MLP / attention block
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers", "5", "--num-layer-list", "[3,2]", "--recompute-module-list", "[2,1]",
         "--recompute-type", "0"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--recompute-module-list", "2,0", "--recompute-type", "1"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--recompute-module-list", "[1,2]"], False),
    # list-valued stage interface with its default content (the one hidden-state tensor), through the plan executor
    (2, ["--pipeline-model-parallel-size", "2", "--use-multiparameter-pipeline-model-parallel"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--recompute-in-advance"], False),
    # interleaved schedule with the first weight-gradient GEMMs of each rank moved behind its last backward
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--use-nanopipe"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--use-nanopipe", "--use-nanopipe-swap"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--schedules-method", "chimera"], True),
    (2, ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipe"], True),
    # receives of the next slot posted before this slot's compute, sends right after it, one communicator per direction
    (2, ["--pipeline-model-parallel-size", "2", "--overlap-p2p-communication"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--overlap-p2p-communication"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipev", "--overlap-p2p-communication"], False),
    (2, ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipe", "--overlap-p2p-communication"], True),
    (4, ["--pipeline-model-parallel-size", "4", "--overlap-p2p-communication"], False),
])
def test_pipeline_matches_no_pipeline(world, extra, bidir):
    # flags that change the model itself also apply to the one-rank oracle
    model_flags = [extra[i + j] for i, x in enumerate(extra) if x in ("--vocab-size", "--num-layers") for j in (0, 1)]
    ref = _reference_losses(tuple(model_flags))
    res = run_distributed(_train, world, extra, bidir)
    have = [r for r in res if r[0] is not None]
    # bidirectional schedules compute half of the micro-batches' losses at each end of the pipeline
    got = [sum(v) / len(v) for v in zip(*have)] if bidir else have[0]
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (ref, got)


def _multi_param(rank, world, overlap):
    """Two stages that hand over (hidden, side tensor, integer positions): gradients of both floating tensors return."""
    import torch.distributed as dist
    import torch.nn as nn
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.pipeline.schedules import get_forward_backward_func
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(pipeline_model_parallel_size=world, optimize_send_recv_comm=overlap)
    cfg = TransformerConfig(num_layers=2, hidden_size=8, num_attention_heads=2, use_cpu_initialization=True, optimization_level=0,
                            pipeline_model_parallel_size=world)
    cfg.pipeline_dtype = torch.float32
    cfg.use_multiparameter_pipeline_model_parallel = True
    cfg.overlap_p2p_comm = overlap
    cfg.pipeline_tensor_shapes = [{"shape": (4, 3), "dtype": torch.float32}, {"shape": (4, 2), "dtype": torch.float32},
                                  {"shape": (4,), "dtype": torch.int64}]
    torch.manual_seed(0)
    lin0, lin_a, lin1, emb = nn.Linear(5, 3), nn.Linear(5, 2), nn.Linear(3, 2), nn.Embedding(7, 2)

    class Stage(nn.Module):
        def __init__(self, first):
            super().__init__()
            self.config, self.first, self.inp = cfg, first, None
            if first:
                self.lin0, self.lin_a = lin0, lin_a
            else:
                self.lin1, self.emb = lin1, emb

        def set_input_tensor(self, t):
            self.inp = t

        def forward(self, x, pos):
            if self.first:
                return self.lin0(x), torch.tanh(self.lin_a(x)), pos
            h, side, p = self.inp
            return ((self.lin1(h) + self.emb(p)) * side).sum()

    data = [(torch.randn(4, 5, generator=torch.Generator().manual_seed(10 + i)), torch.arange(4) + i % 3) for i in range(4)]

    def step(it, model):
        x, pos = next(it)
        out = model(x, pos)
        return out, (lambda o: (o, {"l": o.detach()}))

    # one-process oracle on the same parameters
    ref = {}
    for x, pos in data:
        l = ((lin1(lin0(x)) + emb(pos)) * torch.tanh(lin_a(x))).sum() / len(data)
        l.backward()
    for n, m in (("lin0", lin0), ("lin_a", lin_a), ("lin1", lin1), ("emb", emb)):
        ref[n] = m.weight.grad.clone()
        m.zero_grad()
    model = Stage(first=(rank == 0))
    fb = get_forward_backward_func()
    store = fb(forward_step_func=step, data_iterator=iter(data), model=[model], num_microbatches=len(data), seq_length=4,
               micro_batch_size=1, forward_only=False)
    errs = {}
    for n in (("lin0", "lin_a") if rank == 0 else ("lin1", "emb")):
        errs[n] = (getattr(model, n).weight.grad - ref[n]).abs().max().item()
    ps.destroy_model_parallel()
    dist.destroy_process_group()
    return errs, len(store)


@pytest.mark.parametrize("overlap", [False, True])
def test_multi_parameter_stage_interface(overlap):
    """``--use-multiparameter-pipeline-model-parallel``: stages exchange a list of tensors described by
    ``pipeline_tensor_shapes``; integer entries travel forward only."""
    res = run_distributed(_multi_param, 2, overlap)
    for errs, _ in res:
        for n, e in errs.items():
            assert e < 1e-5, (n, e)
    assert res[1][1] == 4 and res[0][1] == 0        # losses are collected on the last stage
