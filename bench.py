"""Headline benchmark: one pretraining step of a named model/config on N GPUs of one node.

  python bench.py --gpus 1 --steps K --warmup W
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Default model: Llama-3-8B shape, TP = N (+ sequence parallel), bf16 with fp32 master weights, distributed optimizer,
seq 8192, micro-batch 1, global batch 64, synthetic tokens, random init.  ``--model mixtral-8x7b`` runs the Mixtral
shape with EP = N (alltoall dispatcher, TP 1); ``--model llama2-13b`` the long-context CP x TP layout.

Rank 0 prints ONE JSON line.
  value   whole-job tokens/s over the K timed steps (CUDA events, barrier + synchronize on both sides, max over ranks,
          inputs already on the device).
  e2e     the same step through the public training API with every micro-batch copied from pinned host memory and the
          loss read back to the host each step, timed separately over a few steps.
  baseline_arm / vs_baseline
          the same model with library GEMMs (cuBLAS through torch.matmul) and NCCL collectives but this package's
          level-1 elementwise / attention kernels, switched at run time and timed over a few steps.
  fused_comm_check (N > 1)
          one all-gather->GEMM and one GEMM->reduce-scatter of the layer shapes compared with NCCL + fp32 matmul.

The run is bounded by wall-clock time (``--max-seconds``, counted from process start): after the warm-up the step time
is known, and the number of timed steps is cut so the whole run fits; the line then carries ``"truncated": true`` and
the number of steps really timed in ``steps``.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

_T_START = time.time()
ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

UNIT = "tokens/s"
# level-1 kernels + cuBLAS + NCCL on the same box and config, whole-job tokens/s (measured by this script's
# baseline arm; recorded so `vs_baseline` has a fixed denominator when the in-process arm is skipped for time)
RECORDED_BASELINE = {"llama3-8b": {}}


def parse(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--level", type=int, default=int(os.environ.get("MSB200_BENCH_LEVEL", "2")), choices=[0, 1, 2])
    p.add_argument("--model", type=str, default="llama3-8b")
    p.add_argument("--global-batch", type=int, default=None)
    p.add_argument("--seq", type=int, default=None)
    p.add_argument("--num-layers", type=int, default=None, help="override the preset's depth (debug only: reported in config)")
    p.add_argument("--recompute-layers", type=int, default=-1, help="-1: pick by model and GPU count")
    p.add_argument("--max-seconds", type=float, default=float(os.environ.get("MSB200_BENCH_MAX_SECONDS", "660")),
                   help="wall-clock budget of the whole run, counted from process start")
    p.add_argument("--e2e-steps", type=int, default=-1, help="-1: chosen from the step time")
    p.add_argument("--baseline-steps", type=int, default=-1, help="-1: chosen from the step time; 0 disables the arm")
    p.add_argument("--extra", type=str, default="", help="further training flags, space separated (reported in config)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-comm-check", action="store_true")
    p.add_argument("--profile-dir", type=str, default=None,
                   help="run one extra, untimed step under the step-window profiler on rank 0 and write its kernel table here")
    return p.parse_args(argv)


def reference_arm():
    """The reference is an Ascend patch layer over Megatron-LM: it hard-imports torch_npu, every fused op calls
    closed CANN / ATB libraries, and the Megatron checkout it patches is not part of its tree."""
    why = "reference (Ascend/MindSpeed) hard-imports torch_npu + CANN/ATB vendor libraries and patches a Megatron-LM " \
          "checkout that is not shipped with it; it contains no CUDA path and cannot run on a B200"
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    try:
        sys.path.insert(0, ref_dir)
        import importlib
        importlib.import_module("mindspeed.megatron_adaptor")
        why = "reference imported unexpectedly but has no CUDA execution path"
    except Exception as e:  # expected: ModuleNotFoundError torch_npu / megatron
        why += f" (import error: {type(e).__name__}: {str(e)[:80]})"
    finally:
        if ref_dir in sys.path:
            sys.path.remove(ref_dir)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons of this process's GPU with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index, period_ms=200):
        self.index, self.proc, self.lines, self.period_ms = index, None, [], int(period_ms)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # keep samples under load (top half by power) for the median
        if sm:
            thr = statistics.median(power) if power else 0
            load = [s for s, p in zip(sm, power) if p >= thr] or sm
            return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                    "power_w_max": max(power), "samples": len(sm)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


def plan_steps(step_s, budget_left_s, want_steps, want_e2e, want_base, reserve_s=25.0):
    """Split the remaining wall-clock budget into (timed steps, e2e steps, baseline-arm steps).

    ``want_e2e`` / ``want_base`` < 0 mean "choose": two steps each when a step is long, up to five when it is short.
    The baseline arm costs one extra untimed step (its own warm-up).  The timed loop keeps at least two steps; the
    baseline arm is dropped first, then the e2e loop shrinks to one step.  Returns (k, ke, kb, truncated)."""
    afford = int(max(0.0, budget_left_s - reserve_s) / max(step_s, 1e-3))
    auto = 2 if step_s > 2.0 else 5
    ke = min(want_steps, auto) if want_e2e < 0 else want_e2e
    kb = min(want_steps, auto) if want_base < 0 else want_base

    def total(k, ke_, kb_):
        return k + ke_ + (kb_ + 1 if kb_ > 0 else 0)

    k = want_steps
    if total(k, ke, kb) > afford:
        k = max(2, min(want_steps, afford - ke - (kb + 1 if kb > 0 else 0)))
    if total(k, ke, kb) > afford and kb > 0:
        kb = 0
        k = max(2, min(want_steps, afford - ke))
    if total(k, ke, kb) > afford and ke > 1:
        ke = 1
        k = max(2, min(want_steps, afford - ke))
    return k, ke, kb, k < want_steps


def layout_args(a, n):
    """Parallel layout and memory policy of each benchmark config on ``n`` GPUs.  Returns (argument list,
    parallelism string, recompute layers)."""
    rl = a.recompute_layers
    out = ["--use-distributed-optimizer", "--optimization-level", str(a.level)]
    if a.model == "mixtral-8x7b":
        out += ["--expert-model-parallel-size", str(n), "--tensor-model-parallel-size", "1"]
        if a.level >= 2 and n > 1:
            out += ["--moe-alltoall-mc2"]
        par = f"ep{n}+dp{n}+distopt"
        if rl < 0:
            rl = 0
    elif a.model == "llama2-13b":
        tp = 2 if n >= 2 else 1
        cp = max(1, n // tp)
        out += ["--tensor-model-parallel-size", str(tp), "--context-parallel-size", str(cp),
                "--context-parallel-algo", "megatron_cp_algo"]
        if tp > 1:
            out += ["--sequence-parallel"] + (["--use-fused-tp-comm"] if a.level >= 2 else [])
        if cp > 1:
            out += ["--use-cp-send-recv-overlap"]
        par = f"cp{cp}xtp{tp}" + ("+sp" if tp > 1 else "") + "+distopt"
        if rl < 0:
            rl = 40
    else:
        out += ["--tensor-model-parallel-size", str(n)]
        if n > 1:
            out += ["--sequence-parallel"] + (["--use-fused-tp-comm"] if a.level >= 2 else [])
        if n == 1:
            # one GPU holds the whole model: keep the master weights as (bf16 parameter + 16-bit residual) to
            # free 16 GB for activations
            out += ["--reuse-fp32-param"]
        par = f"tp{n}" + ("+sp" if n > 1 else "") + "+distopt"
        if rl < 0:
            rl = {1: 8}.get(n, 0)
    if rl > 0:
        out += ["--recompute-granularity", "full", "--recompute-method", "block", "--recompute-num-layers", str(rl)]
    return out, par, rl


def fused_comm_check(args, dev):
    """One all-gather->GEMM and one GEMM->reduce-scatter of the QKV / FC2 layer shapes against NCCL + fp32 matmul.
    Returns {max_rel_err, deterministic, shapes}; run on every rank (collective)."""
    import torch
    import torch.distributed as dist
    from mindspeed_b200.ops.fused_comm import FusedOps
    from mindspeed_b200.parallel import mappings as M
    from mindspeed_b200.parallel import parallel_state as ps
    g = ps.get_tensor_model_parallel_group()
    ws = dist.get_world_size(g)
    s, h, f = args.seq_length, args.hidden_size, args.ffn_hidden_size
    gen = torch.Generator(device=dev).manual_seed(4321 + dist.get_rank(g))
    res = {"max_rel_err": 0.0, "deterministic": True, "shapes": []}

    def rel(a, b):
        return float((a.float() - b).abs().max() / b.abs().max().clamp(min=1e-6))

    # all-gather -> GEMM (column-parallel fc1 shape): x [s/ws, h], w [2f/ws, h]
    x = torch.randn(s // ws, h, device=dev, dtype=torch.bfloat16, generator=gen)
    w = torch.randn(2 * f // ws, h, device=dev, dtype=torch.bfloat16, generator=gen) * 0.02
    y1, _ = FusedOps.allgather_matmul(x, w, g, nt=True)
    y2, _ = FusedOps.allgather_matmul(x, w, g, nt=True)
    ref = M.all_gather_first_dim(x, g).float() @ w.float().t()
    res["max_rel_err"] = max(res["max_rel_err"], rel(y1, ref))
    res["deterministic"] &= bool(torch.equal(y1, y2))
    res["shapes"].append(["ag_gemm", s, 2 * f // ws, h])
    # GEMM -> reduce-scatter (row-parallel fc2 shape): x [s, f/ws], w [h, f/ws]
    x = torch.randn(s, f // ws, device=dev, dtype=torch.bfloat16, generator=gen)
    w = torch.randn(h, f // ws, device=dev, dtype=torch.bfloat16, generator=gen) * 0.02
    z1 = FusedOps.matmul_reduce_scatter(x, w, g, nt=True).clone()
    z2 = FusedOps.matmul_reduce_scatter(x, w, g, nt=True)
    part = (x.float() @ w.float().t())
    ref = torch.empty(s // ws, h, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(ref, part, group=g)
    res["max_rel_err"] = max(res["max_rel_err"], rel(z1, ref))
    res["deterministic"] &= bool(torch.equal(z1, z2))
    res["shapes"].append(["gemm_rs", s, h, f // ws])
    t = torch.tensor([res["max_rel_err"], 0.0 if res["deterministic"] else 1.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["max_rel_err"], res["deterministic"] = float(t[0]), bool(t[1] == 0)
    return res


def main(argv=None):
    a = parse(argv)
    if a.impl == "reference":
        return reference_arm()
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    import torch
    import torch.distributed as dist
    import pretrain_gpt as pg
    from mindspeed_b200.models.presets import PRESETS
    from mindspeed_b200.ops import gemm as G
    from mindspeed_b200.ops import loader
    from mindspeed_b200.parallel import comm_ops
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.training import flops as flops_mod
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import BatchIterator, SyntheticGPTDataset

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    n = a.gpus
    kw = {}
    if a.seq is not None:
        kw["seq"] = a.seq
    if a.global_batch is not None:
        kw["gbs"] = a.global_batch
    args_list = PRESETS[a.model](**kw)
    lay, par, rl = layout_args(a, n)
    args_list += lay + ["--train-iters", "1000000", "--log-interval", "1000000"] + a.extra.split()
    if a.num_layers is not None:
        i = args_list.index("--num-layers")
        args_list[i + 1] = str(a.num_layers)
    args = initialize_megatron(args_list=args_list)
    dev = torch.device("cuda", torch.cuda.current_device())
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
    dp_r, dp_n = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
    nmb = args.global_batch_size // (args.micro_batch_size * dp_n)

    # one step's micro-batches, generated once on the host (pinned) and cycled by both iterators
    src = BatchIterator(ds, args.micro_batch_size, dp_r, dp_n, pin=True)
    host_batches = [next(src) for _ in range(nmb)]
    h2d_bytes = sum(v.numel() * v.element_size() for b in host_batches for v in b.values())

    class Cycle:
        def __init__(self, batches):
            self.b, self.i = batches, 0

        def __iter__(self):
            return self

        def __next__(self):
            x = self.b[self.i % len(self.b)]
            self.i += 1
            return x

    dev_iter = Cycle([{k: v.to(dev) for k, v in b.items()} for b in host_batches])   # device-resident inputs
    host_iter = Cycle(host_batches)                                                  # pinned host inputs, copied per step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(k, it, read_loss):
        last = None
        for _ in range(k):
            ld, _, _, _ = train_step(pg.forward_step, it, model, opt, sched)
            if read_loss:
                last = float(ld["lm loss"]) if "lm loss" in ld else None  # device -> host read of the step result
        return last

    def timed(k, it, read_loss):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        last = run(k, it, read_loss)
        e1.record()
        barrier()
        G.check_status()          # a bounded wait that expired inside the region invalidates the number
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), last

    comm_check = None
    if n > 1 and a.level >= 2 and not a.no_comm_check and ps.get_tensor_model_parallel_world_size() > 1:
        comm_check = fused_comm_check(args, dev)
        G.check_status()

    # ---- warm-up: W steps, the last one timed to learn the step time ----
    run(max(a.warmup - 1, 0), dev_iter, False)
    step_ms, _ = timed(1, dev_iter, False) if a.warmup >= 1 else (0.0, None)
    if a.profile_dir and rank == 0:
        from mindspeed_b200.utils.profiler import StepWindowProfiler
        with StepWindowProfiler(start=0, end=1, save_path=a.profile_dir, rank=0, level="level0") as prof:
            run(1, dev_iter, False)
            prof.step()
    elif a.profile_dir:
        run(1, dev_iter, False)          # the other ranks take part in the profiled step's collectives
    budget_left = a.max_seconds - (time.time() - _T_START)
    plan = torch.tensor(list(plan_steps(step_ms / 1e3, budget_left, a.steps, 0 if a.no_e2e else a.e2e_steps,
                                        a.baseline_steps if a.level >= 1 else 0)), device=dev, dtype=torch.int64)
    if world > 1:
        dist.broadcast(plan, src=0)      # every rank must run the same number of steps
    k, ke, kb, truncated = (int(x) for x in plan.tolist())

    # ---- the timed region: exactly k steps, device-resident inputs ----
    # 200 ms samples; 500 ms once a step takes seconds (still several samples per step, fewer driver queries beside a
    # model that synchronises with the host in every layer)
    sampler = ClockSampler(torch.cuda.current_device(), 200 if step_ms < 2000 else 500)
    barrier()
    if rank == 0:
        sampler.start()
    loader.reset_launch_count()
    ms_total, _ = timed(k, dev_iter, False)
    launches = loader.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    tokens_per_step = args.global_batch_size * args.seq_length
    value = k * tokens_per_step / (ms_total / 1e3)

    # ---- end to end: pinned host inputs copied every micro-batch, loss read back every step ----
    e2e = None
    if ke > 0:
        ms2, last_loss = timed(ke, host_iter, True)
        e2e = {"value": ke * tokens_per_step / (ms2 / 1e3), "unit": UNIT, "steps": ke, "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 8, "last_loss": last_loss}

    # ---- baseline arm: same model, library GEMM + NCCL collectives, this package's elementwise/attention kernels ----
    base = None
    if kb > 0:
        prev = comm_ops.get_ops()
        comm_ops.set_ops(comm_ops.DefaultOps)
        try:
            run(1, dev_iter, False)
            ms3, _ = timed(kb, dev_iter, False)
            base = {"value": kb * tokens_per_step / (ms3 / 1e3), "unit": UNIT, "steps": kb,
                    "what": "level-1 kernels + cuBLAS (torch.matmul) + NCCL, switched in process"}
        finally:
            comm_ops.set_ops(prev)

    if rank == 0:
        step_s = ms_total / 1e3 / k
        f_model = flops_mod.num_floating_point_operations(args, args.global_batch_size)
        f_hw = f_model + flops_mod.recompute_extra_flops(args, args.global_batch_size)
        peaks = flops_mod.measured_peaks()
        rec = RECORDED_BASELINE.get(a.model, {}).get(n)
        denom = base["value"] if base else rec
        out = {"metric": f"tokens/sec (whole job; /GPU and MFU alongside), {a.model}-shape {par} bf16", "value": value, "unit": UNIT,
               "n_gpus": n, "steps": k, "warmup": a.warmup, "ms_per_step": ms_total / k, "higher_is_better": True,
               "scaling": "strong", "vs_baseline": (value / denom) if denom else None,
               "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
               "tokens_per_sec_per_gpu": value / n,
               "mfu_of_measured_bf16_peak": f_model / (step_s * n * peaks["bf16_tflops"] * 1e12),
               "hfu_of_measured_bf16_peak": f_hw / (step_s * n * peaks["bf16_tflops"] * 1e12),
               "mfu_of_sustained_bf16_peak": f_model / (step_s * n * peaks["bf16_tflops_sustained"] * 1e12),
               "config": {"model": a.model, "global_batch": args.global_batch_size, "seq_len": args.seq_length,
                          "micro_batch": args.micro_batch_size, "num_layers": args.num_layers, "parallelism": par,
                          "optimization_level": a.level, "recompute_layers": rl, "extra_flags": a.extra,
                          "reuse_fp32_param": bool(getattr(args, "reuse_fp32_param", False)),
                          "same_config_for_all_n": "no: one GPU recomputes 8 layers and packs the fp32 masters to fit 180 GB; "
                                                   "hfu_of_measured_bf16_peak counts the recomputed FLOPs",
                          "l2": "per-step working set (>= 2 GB of weights per GPU) far exceeds the 126 MB L2"},
               "clocks": clocks, "e2e": e2e, "baseline_arm": base, "fused_comm_check": comm_check,
               "truncated": bool(truncated), "requested_steps": a.steps, "budget_s": a.max_seconds,
               "projected_s": round((time.time() - _T_START), 1), "warmup_step_ms": step_ms,
               "gpu_launches": int(launches), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
               "impl": "ours"}
        print(json.dumps(out))
        sys.stdout.flush()
    if world > 1:
        dist.barrier()
    if dist.is_initialized():
        from mindspeed_b200.parallel.symm_mem import destroy_heaps
        destroy_heaps()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
