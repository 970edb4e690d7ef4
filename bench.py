"""Headline benchmark: Llama-3-8B-shape pretraining step, TP = N (+ sequence parallel), bf16 with fp32 master
weights, distributed optimizer, seq 8192, micro-batch 1, global batch 64, synthetic tokens, random init.

  python bench.py --gpus 1 --steps K --warmup W
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Prints one JSON line on rank 0.  ``value`` = whole-job tokens/s measured with CUDA events around exactly K
steps (barrier + synchronize on both sides, max over ranks), inputs pre-staged on the device.  ``e2e`` = the same
K steps through the public training API with every micro-batch copied from pinned host memory and the loss read
back to the host each step.  ``--impl reference`` reports why the reference cannot run here.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "tokens/sec (whole job), Llama-3-8B-shape TP=N SP bf16"
UNIT = "tokens/s"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--level", type=int, default=int(os.environ.get("MSB200_BENCH_LEVEL", "2")), choices=[0, 1, 2])
    p.add_argument("--model", type=str, default="llama3-8b")
    p.add_argument("--global-batch", type=int, default=64)
    p.add_argument("--seq", type=int, default=8192)
    p.add_argument("--recompute-layers", type=int, default=-1, help="-1: pick by GPU count")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--profile-dir", type=str, default=None,
                   help="run one extra, untimed step under the step-window profiler on rank 0 and write its kernel table here")
    return p.parse_args()


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

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
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


def main():
    a = parse()
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
    from mindspeed_b200.ops import loader
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.training import flops as flops_mod
    from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
    from mindspeed_b200.training.data import BatchIterator, SyntheticGPTDataset

    world = int(os.environ["WORLD_SIZE"])
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    n = a.gpus
    args_list = PRESETS[a.model](seq=a.seq, gbs=a.global_batch)
    args_list += ["--tensor-model-parallel-size", str(n), "--use-distributed-optimizer", "--optimization-level", str(a.level),
                  "--train-iters", str(a.steps + a.warmup + a.steps), "--log-interval", "1000000"]
    if n > 1:
        args_list += ["--sequence-parallel"]
        if a.level >= 2:
            args_list += ["--use-fused-tp-comm"]
    rl = a.recompute_layers
    if n == 1:
        # one GPU holds the whole model: keep the master weights as (bf16 parameter + 16-bit residual) to free 16 GB for activations
        args_list += ["--reuse-fp32-param"]
    if rl < 0:
        rl = {1: 8}.get(n, 0)
    if rl > 0:
        args_list += ["--recompute-granularity", "full", "--recompute-method", "block", "--recompute-num-layers", str(rl)]
    args = initialize_megatron(args_list=args_list)
    dev = torch.device("cuda", torch.cuda.current_device())
    model, opt, sched = setup_model_and_optimizer(pg.model_provider)
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
    dp_r, dp_n = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
    nmb = args.global_batch_size // (args.micro_batch_size * dp_n)

    # device-resident data for the device-timed number: one step's micro-batches, cycled
    class DeviceIter:
        def __init__(self):
            it = BatchIterator(ds, args.micro_batch_size, dp_r, dp_n)
            self.batches = [{k: v.to(dev) for k, v in next(it).items()} for _ in range(nmb)]
            self.i = 0

        def __iter__(self):
            return self

        def __next__(self):
            b = self.batches[self.i % len(self.batches)]
            self.i += 1
            return b

    dev_iter = DeviceIter()
    host_iter = BatchIterator(ds, args.micro_batch_size, dp_r, dp_n, pin=True)

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

    run(a.warmup, dev_iter, False)
    if a.profile_dir and int(os.environ["RANK"]) == 0:
        from mindspeed_b200.utils.profiler import StepWindowProfiler
        with StepWindowProfiler(start=0, end=1, save_path=a.profile_dir, rank=0, level="level0") as prof:
            run(1, dev_iter, False)
            prof.step()
    elif a.profile_dir:
        run(1, dev_iter, False)          # the other ranks take part in the profiled step's collectives
    sampler = ClockSampler(torch.cuda.current_device())
    barrier()
    if int(os.environ["RANK"]) == 0:
        sampler.start()
    loader.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    h0 = time.perf_counter()
    run(a.steps, dev_iter, False)
    host_enqueue_ms = (time.perf_counter() - h0) * 1e3     # host time to queue the steps; ~ device time means launch-bound
    e1.record()
    barrier()
    launches = loader.launch_count()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop() if int(os.environ["RANK"]) == 0 else None

    e2e = None
    if not a.no_e2e:
        run(1, host_iter, True)
        barrier()
        e0.record()
        last_loss = run(a.steps, host_iter, True)
        e1.record()
        barrier()
        ms2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        tok = a.steps * args.global_batch_size * args.seq_length
        per_mb = sum(v.numel() * v.element_size() for v in next(BatchIterator(ds, args.micro_batch_size, dp_r, dp_n)).values())
        e2e = {"value": tok / (float(ms2.item()) / 1e3), "unit": UNIT, "h2d_bytes_per_step": per_mb * nmb,
               "d2h_bytes_per_step": 8, "last_loss": last_loss}

    if int(os.environ["RANK"]) == 0:
        tokens = a.steps * args.global_batch_size * args.seq_length
        value = tokens / (ms_total / 1e3)
        step_s = ms_total / 1e3 / a.steps
        out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": a.steps, "warmup": a.warmup,
               "ms_per_step": ms_total / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
               "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
               "tokens_per_sec_per_gpu": value / n,
               "mfu_of_measured_bf16_peak": flops_mod.mfu(args, args.global_batch_size, step_s, n),
               "config": {"model": a.model, "global_batch": args.global_batch_size, "seq_len": args.seq_length,
                          "micro_batch": args.micro_batch_size, "parallelism": f"tp{n}" + ("+sp" if n > 1 else "") + "+distopt",
                          "optimization_level": a.level, "recompute_layers": rl,
                          "l2": "per-step working set (>= 2 GB of weights per GPU) far exceeds the 126 MB L2"},
               "clocks": clocks, "e2e": e2e, "host_enqueue_ms_per_step": host_enqueue_ms / a.steps, "gpu_launches": int(launches), "impl": "ours"}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
    if dist.is_initialized():
        from mindspeed_b200.parallel.symm_mem import destroy_heaps
        destroy_heaps()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
