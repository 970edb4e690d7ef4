"""Measured pipeline bubble against the analytic one, per schedule.

Run one process per pipeline stage:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29800 \
        -m mindspeed_b200.benchmarks.microbench_pipeline --schedules 1f1b,1f1b_overlap,dualpipev,dualpipev_overlap

The forward-backward function of each schedule (no optimizer step) is timed with CUDA events at two micro-batch counts
n1 < n2.  In steady state every extra micro-batch costs the same ``t_mb``, so ``t_mb = (T(n2) - T(n1)) / (n2 - n1)`` and the
time lost to fill / drain at n1 is ``T(n1) - n1 * t_mb``: the measured bubble fraction is that over ``T(n1)``.  The analytic
figure comes from the schedule's own plan, simulated with unit costs F = 1, B = 2 (B = W = 1 when the schedule splits the
weight gradient).  Reference: the schedules of mindspeed/core/pipeline_parallel/dualpipev/dualpipev_schedules.py:310-346
and Megatron's 1F1B, whose bubble is (p - 1) / (n + p - 1).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _args_list(pp, n, extra, hidden, layers, seq):
    return ["--num-layers", str(layers), "--hidden-size", str(hidden), "--num-attention-heads", str(hidden // 128),
            "--group-query-attention", "--num-query-groups", str(max(1, hidden // 512)), "--ffn-hidden-size", str(hidden * 7 // 2),
            "--seq-length", str(seq), "--max-position-embeddings", str(seq), "--micro-batch-size", "1", "--global-batch-size",
            str(n), "--vocab-size", "32768", "--make-vocab-size-divisible-by", "1", "--bf16", "--lr", "1e-4", "--lr-decay-style",
            "constant", "--hidden-dropout", "0", "--attention-dropout", "0", "--swiglu", "--normalization", "RMSNorm",
            "--position-embedding-type", "rope", "--disable-bias-linear", "--untie-embeddings-and-output-weights",
            "--use-flash-attn", "--train-iters", "100", "--optimization-level", "2", "--pipeline-model-parallel-size", str(pp)] + extra


SCHEDULES = {
    "1f1b": [],
    "1f1b_overlap": ["--overlap-p2p-communication"],
    "interleaved_overlap": ["--num-layers-per-virtual-pipeline-stage", "LPV", "--overlap-p2p-communication"],
    "dualpipev": ["--schedules-method", "dualpipev"],
    "dualpipev_overlap": ["--schedules-method", "dualpipev", "--overlap-p2p-communication"],
}


def analytic_bubble(name, pp, n):
    from ..parallel.pipeline.plan import order_dualpipev, order_interleaved, placement_interleaved, placement_v, simulate_orders
    if name.startswith("1f1b"):
        return (pp - 1) / (n + pp - 1)
    if name.startswith("dualpipev"):
        _, b = simulate_orders(placement_v(pp), order_dualpipev(pp, n, True), {"F": 1, "B": 1, "W": 1})
        return b
    _, b = simulate_orders(placement_interleaved(pp, 2), order_interleaved(pp, 2, n), {"F": 1, "B": 2, "W": 0})
    return b


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--schedules", default="1f1b,1f1b_overlap,dualpipev,dualpipev_overlap")
    ap.add_argument("--n1", type=int, default=8)
    ap.add_argument("--n2", type=int, default=24)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    pp = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    sys.path.insert(0, os.getcwd())
    import pretrain_gpt as pg
    from ..parallel import parallel_state as ps
    from ..parallel.pipeline.schedules import get_forward_backward_func
    from ..training import initialize_megatron, setup_model_and_optimizer
    from ..training.data import BatchIterator, SyntheticGPTDataset
    rows = []
    model = None
    for name in a.schedules.split(","):
        extra = [str(a.layers // pp // 2) if x == "LPV" else x for x in SCHEDULES[name]]
        if model is not None:
            del model, opt, sched
            from ..parallel.symm_mem import destroy_heaps
            destroy_heaps()
            ps.destroy_model_parallel()
            torch.cuda.empty_cache()
        args = initialize_megatron(args_list=_args_list(pp, a.n1, extra, a.hidden, a.layers, a.seq))
        dev = torch.device("cuda", torch.cuda.current_device())
        model, opt, sched = setup_model_and_optimizer(pg.model_provider)
        ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 256, seed=1)
        batch = {k: v.to(dev) for k, v in next(BatchIterator(ds, 1, 0, 1)).items()}

        class Same:
            def __iter__(self):
                return self

            def __next__(self):
                return batch

        it = Same()
        fb = get_forward_backward_func()

        def step(n):
            args.global_batch_size = n               # one data-parallel replica: micro-batches per step = global batch
            for m in model:
                m.zero_grad_buffer()
            fb(forward_step_func=pg.forward_step, data_iterator=[it] * len(model) if len(model) > 1 else it, model=model,
               num_microbatches=n, seq_length=args.seq_length, micro_batch_size=1, decoder_seq_length=None, forward_only=False)

        def timed(n):
            step(n)                                           # warm-up at this count
            best = None
            for _ in range(a.reps):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step(n)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                best = float(t) if best is None else min(best, float(t))
            return best

        t1, t2 = timed(a.n1), timed(a.n2)
        t_mb = (t2 - t1) / (a.n2 - a.n1)
        row = {"schedule": name, "pp": pp, "n1": a.n1, "n2": a.n2, "T_n1_ms": t1, "T_n2_ms": t2, "t_mb_ms": t_mb,
               "bubble_measured_n1": 1.0 - a.n1 * t_mb / t1, "bubble_analytic_n1": analytic_bubble(name, pp, a.n1),
               "bubble_measured_n2": 1.0 - a.n2 * t_mb / t2, "bubble_analytic_n2": analytic_bubble(name, pp, a.n2)}
        rows.append(row)
        if rank == 0:
            print(f"pipeline pp={pp} {name:20s} T({a.n1})={t1:8.1f} ms  T({a.n2})={t2:8.1f} ms  per-mb {t_mb:7.2f} ms  "
                  f"bubble n={a.n1}: measured {row['bubble_measured_n1']:.3f} analytic {row['bubble_analytic_n1']:.3f}", flush=True)
    if rank == 0 and a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    from ..parallel.symm_mem import destroy_heaps
    destroy_heaps()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
