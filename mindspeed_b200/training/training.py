"""pretrain() / train() / train_step() (Megatron ``training`` surface).

reference: mindspeed/training.py:78-160 (train_step with EMA update), :163-384 (pretrain),
mindspeed/functional/profile/adaptor.py:13-78 (profiler wrapping), tflops logging
mindspeed/functional/tflops_calculate/adaptor.py:196-231.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from ..optimizer import OptimizerConfig, get_megatron_optimizer
from ..parallel import parallel_state as ps
from ..parallel.distributed import DistributedDataParallel, DistributedDataParallelConfig, finalize_model_grads
from ..parallel.pipeline.schedules import get_forward_backward_func
from ..utils.logging import print_rank_0, print_rank_last
from . import flops as flops_mod
from .global_vars import get_args, get_num_microbatches, get_timers
from .initialize import initialize_megatron


class OptimizerParamScheduler:
    """Learning-rate schedule: warmup then constant / linear / cosine / inverse-sqrt decay."""

    def __init__(self, optimizer, max_lr, min_lr, warmup_steps, decay_steps, style, start_wd=None, end_wd=None, wd_incr_steps=0,
                 wd_incr_style="constant"):
        self.opt, self.max_lr, self.min_lr = optimizer, max_lr, min_lr
        self.warmup, self.decay, self.style, self.num_steps = warmup_steps, decay_steps, style, 0
        # weight decay moves from start_wd to end_wd over wd_incr_steps (--start/--end-weight-decay, --weight-decay-incr-style)
        self.start_wd, self.end_wd, self.wd_steps, self.wd_style = start_wd, end_wd, wd_incr_steps, wd_incr_style
        self.step(0)

    def get_wd(self):
        if self.start_wd is None or self.wd_style == "constant" or not self.wd_steps:
            return self.end_wd
        r = min(1.0, self.num_steps / self.wd_steps)
        c = r if self.wd_style == "linear" else 0.5 * (math.cos(math.pi * (1.0 - r)) + 1.0)
        return self.start_wd + c * (self.end_wd - self.start_wd)

    def get_lr(self):
        n = self.num_steps
        if self.warmup > 0 and n <= self.warmup:
            return self.max_lr * n / self.warmup
        if self.style == "constant" or not self.decay:
            return self.max_lr
        if n > self.decay:
            return self.min_lr
        r = (n - self.warmup) / max(1, self.decay - self.warmup)
        if self.style == "linear":
            c = 1.0 - r
        elif self.style == "cosine":
            c = 0.5 * (math.cos(math.pi * r) + 1.0)
        elif self.style == "inverse-square-root":
            return max(self.min_lr, self.max_lr * math.sqrt(max(self.warmup, 1)) / math.sqrt(max(n, 1)))
        else:
            c = 1.0
        return self.min_lr + c * (self.max_lr - self.min_lr)

    def step(self, increment=1):
        self.num_steps += increment
        lr = self.get_lr()
        wd = self.get_wd()
        scheduled = wd is not None and self.wd_style != "constant"
        for g in self.opt.param_groups:
            g["lr"] = lr
            if scheduled and "weight_decay" in g:
                # groups that were built without decay (biases, norm gains in torch-style optimizers) stay without
                if g.setdefault("wd_scheduled", g["weight_decay"] != 0.0 or self.start_wd == 0.0 and len(self.opt.param_groups) == 1):
                    g["weight_decay"] = wd

    def state_dict(self):
        return {"num_steps": self.num_steps,
                "schedule": {k: getattr(self, k) for k in ("max_lr", "min_lr", "warmup", "decay", "style", "start_wd", "end_wd",
                                                           "wd_steps", "wd_style")}}

    def load_state_dict(self, sd):
        self.num_steps = sd["num_steps"]
        self.step(0)


def get_model(model_provider_func, wrap_with_ddp=True):
    args = get_args()
    vpp = ps.get_virtual_pipeline_model_parallel_world_size()
    models = []
    pp = ps.get_pipeline_model_parallel_world_size()
    if pp > 1 and args.schedules_method in ("dualpipe", "chimera"):
        # bidirectional: chunk 0 is stage r of the "down" replica, chunk 1 is stage pp-1-r of the "up" replica
        r = ps.get_pipeline_model_parallel_rank()
        models.append(model_provider_func(pre_process=(r == 0), post_process=(r == pp - 1)))
        ps.set_pipeline_model_parallel_rank(pp - 1 - r)
        try:
            models.append(model_provider_func(pre_process=(pp - 1 - r == 0), post_process=(pp - 1 - r == pp - 1)))
        finally:
            ps.set_pipeline_model_parallel_rank(None)
    elif pp > 1 and (vpp is not None or args.schedules_method in ("dualpipev",)):
        n = vpp if vpp is not None else 2
        if vpp is None:
            ps.set_virtual_pipeline_model_parallel_world_size(2)
        for i in range(n):
            ps.set_virtual_pipeline_model_parallel_rank(i)
            if args.schedules_method == "dualpipev":
                # V shape: chunk 0 is the head on pp rank 0, chunk 1 is the tail on pp rank 0
                pre = ps.get_pipeline_model_parallel_rank() == 0 and i == 0
                post = ps.get_pipeline_model_parallel_rank() == 0 and i == 1
            else:
                pre, post = ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()
            models.append(model_provider_func(pre_process=pre, post_process=post))
        ps.set_virtual_pipeline_model_parallel_rank(0)
    else:
        models.append(model_provider_func(pre_process=ps.is_pipeline_first_stage(), post_process=ps.is_pipeline_last_stage()))
    for m in models:
        if torch.cuda.is_available() and dist.get_backend() != "gloo":
            m.cuda(torch.cuda.current_device())
    if not wrap_with_ddp:
        return models
    cfg = models[0].config
    if getattr(args, "layerzero", False) or getattr(args, "fsdp2_config_path", None):
        # fully sharded data parallel instead of bucketed DDP (+ optional ZeRO-1 of the optimizer state across replicas)
        if pp > 1 and not args.untie_embeddings_and_output_weights:
            raise NotImplementedError("--layerzero / --fsdp2-config-path with pipeline parallelism need "
                                      "--untie-embeddings-and-output-weights (a tied weight lives on two stages)")
        from ..parallel.distributed.fsdp import FSDPPlan, FullyShardedDataParallel
        path = getattr(args, "fsdp2_config_path", None) or getattr(args, "layerzero_config", None)
        plan = FSDPPlan.from_yaml(path) if path else FSDPPlan(zero1_over_replicas=bool(getattr(args, "layerzero", False)))
        ranks = ps._ranks("dp")
        # group creation is collective over the job: every rank creates the shard / replica groups of every data-parallel
        # group (one per tensor- and pipeline-parallel coordinate) in the same order; chunks of one rank share theirs
        from ..parallel.distributed.fsdp import build_groups
        shard_g, rep_g = build_groups(ranks, plan.shard_size, ps.get_all_ranks("dp"))
        if shard_g is None and rep_g is None and len(ranks) == 1:
            shard_g = "local"
        return [FullyShardedDataParallel(m, plan, dp_group_ranks=ranks, shard_group=shard_g, replica_group=rep_g) for m in models]
    ddp_cfg = DistributedDataParallelConfig(
        grad_reduce_in_fp32=args.accumulate_allreduce_grads_in_fp32, overlap_grad_reduce=args.overlap_grad_reduce,
        quant_grads=bool(getattr(args, "quant_grads", False)),
        overlap_param_gather=args.overlap_param_gather, use_distributed_optimizer=args.use_distributed_optimizer,
        check_for_nan_in_grad=args.check_for_nan_in_loss_and_grad, bucket_size=args.ddp_bucket_size,
        average_in_collective=args.ddp_average_in_collective, param_and_grad_buffer_pad=args.param_and_grad_buffer_pad,
        num_distributed_optimizer_instances=args.num_distributed_optimizer_instances,
        fused_dist_opt=bool(getattr(args, "use_fused_dist_opt", False) and args.use_distributed_optimizer
                            and getattr(args, "optimization_level", 0) >= 2 and torch.cuda.is_available()))
    models = [DistributedDataParallel(cfg, ddp_cfg, m, disable_bucketing=(i > 0)) for i, m in enumerate(models)]
    return models


def setup_model_and_optimizer(model_provider_func, no_wd_decay_cond=None, scale_lr_cond=None, lr_mult=1.0):
    args = get_args()
    model = get_model(model_provider_func)
    if no_wd_decay_cond is None and getattr(args, "apply_wd_to_qk_layernorm", False):
        # default rule (no decay on biases and 1-D tensors) except that the q / k layer-norm gains do decay
        def no_wd_decay_cond(name, p):
            if "q_layernorm" in name or "k_layernorm" in name:
                return False
            return name.endswith(".bias") or p.dim() == 1
    ocfg = OptimizerConfig(optimizer=args.optimizer, lr=args.lr, min_lr=args.min_lr, weight_decay=args.weight_decay,
                           bf16=args.bf16, fp16=args.fp16, params_dtype=args.params_dtype, adam_beta1=args.adam_beta1,
                           adam_beta2=args.adam_beta2, adam_eps=args.adam_eps, clip_grad=args.clip_grad,
                           use_distributed_optimizer=args.use_distributed_optimizer,
                           optimizer_selection=args.optimizer_selection, use_ema=args.use_ema, ema_decay=args.ema_decay,
                           swap_optimizer=args.swap_optimizer, swap_optimizer_times=args.swap_optimizer_times,
                           quant_states=args.quant_states, reuse_fp32_param=args.reuse_fp32_param,
                           compress_optimizer=bool(getattr(args, "compress_optimizer", False)))
    from ..parallel.distributed.fsdp import FullyShardedDataParallel as _FSDP
    if isinstance(model[0], _FSDP):
        from ..parallel.distributed.fsdp import ShardedAdamW
        optimizer = ShardedAdamW(model, lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                                 weight_decay=args.weight_decay, clip_grad=args.clip_grad)
    else:
        optimizer = get_megatron_optimizer(ocfg, model, no_wd_decay_cond, scale_lr_cond, lr_mult)
    decay_iters = args.lr_decay_iters or args.train_iters
    warmup = args.lr_warmup_iters
    if getattr(args, "lr_warmup_fraction", None) is not None:
        warmup = int(args.lr_warmup_fraction * decay_iters)          # --lr-warmup-fraction overrides --lr-warmup-iters
    sched = OptimizerParamScheduler(optimizer, args.lr, args.min_lr, warmup, decay_iters, args.lr_decay_style,
                                    start_wd=getattr(args, "start_weight_decay", None), end_wd=getattr(args, "end_weight_decay", None),
                                    wd_incr_steps=args.train_iters or 0, wd_incr_style=getattr(args, "weight_decay_incr_style", "constant"))
    cfg = model[0].module.config
    cfg.finalize_model_grads_func = finalize_model_grads
    if args.swap_attention:
        from ..memory.swap_attention import install_swap_attention
        install_swap_attention(model, args)
    if getattr(args, "te_comparison_with_bf16", False) or getattr(args, "te_comparison_with_cpu", False):
        from ..models.te_compat import OnlineComparison
        OnlineComparison.configure(with_bf16=args.te_comparison_with_bf16, with_cpu=args.te_comparison_with_cpu)
    if getattr(args, "qat_scheme", None):
        from ..qat import QATConfig, apply_qat
        qcfg = QATConfig(scheme=args.qat_scheme.upper(), weight_group=getattr(args, "qat_quant_block_size", 128))
        for m in model:
            apply_qat(m, qcfg)
    if getattr(args, "qad_enable", False):
        from ..qat.qad import setup_teacher
        setup_teacher(model_provider_func, args)      # full precision, frozen; not touched by --qat-scheme
    _MEMORY_MANAGERS.clear()
    _MEMORY_MANAGERS.extend(build_memory_managers(args, model))
    if args.load and getattr(args, "finetune", False):
        from ..qat.qad import load_model_weights
        load_model_weights(model, args.load)
        for chunk in model:
            if hasattr(chunk, "post_load"):
                chunk.post_load()
        if hasattr(optimizer, "reload_model_params"):
            optimizer.reload_model_params()
        args.iteration = 0
    elif args.load:
        from ..checkpointing import load_checkpoint
        args.iteration = load_checkpoint(model, optimizer, sched)
    else:
        args.iteration = 0
    return model, optimizer, sched


_MEMORY_MANAGERS = []   # objects with step_context() / end_step(): smart swap, adaptive recompute


def build_memory_managers(args, model):
    """Per-step memory policies selected by flags.  Each wraps the forward/backward of a step in a context manager
    (profiling or executing its policy through saved-tensor hooks) and is told when the step ends."""
    out = []
    budget_mb = getattr(args, "adaptive_recompute_device_size", -1)
    dev_swap = bool(getattr(args, "adaptive_recompute_device_swap", False))
    if getattr(args, "adaptive_memory_optimization", False) and not getattr(args, "smart_swap", False):
        # recompute / host swap / keep chosen per module from a profile (memory/adaptive_memory.py)
        from ..memory.adaptive_memory import AdaptiveMemory
        pp = ps.get_pipeline_model_parallel_world_size()
        in_flight = 1 if pp <= 1 else min(pp - ps.get_pipeline_model_parallel_rank(), get_num_microbatches())
        for m in model:
            out.append(AdaptiveMemory(m, profiling_steps=getattr(args, "adaptive_recompute_profiling_step", 10),
                                      device_budget_bytes=(budget_mb << 20) if budget_mb and budget_mb > 0 else None,
                                      in_flight=in_flight))
    elif ((budget_mb and budget_mb > 0) or dev_swap) and not getattr(args, "smart_swap", False):
        from ..memory.adaptive_recompute import AdaptiveRecompute
        for m in model:
            out.append(AdaptiveRecompute(m, profiling_steps=getattr(args, "adaptive_recompute_profiling_step", 10),
                                         device_budget_bytes=(budget_mb << 20) if budget_mb and budget_mb > 0 else None,
                                         swap_while_profiling=dev_swap))
    if getattr(args, "smart_swap", False):
        from ..memory.smart_swap import SmartSwapManager
        if torch.cuda.is_available():
            total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
            budget = int(0.85 * total) if not (budget_mb and budget_mb > 0) else budget_mb << 20
        else:
            budget = (budget_mb << 20) if budget_mb and budget_mb > 0 else 1 << 40
        out.append(SmartSwapManager(budget_bytes=budget, warmup_steps=2))
    return out


def train_step(forward_step_func, data_iterator, model, optimizer, opt_param_scheduler, config=None):
    """One optimizer step over ``num_microbatches`` micro-batches."""
    import contextlib as _cl
    with _cl.ExitStack() as _stack:
        for mgr in _MEMORY_MANAGERS:
            _stack.enter_context(mgr.step_context())
        out = _train_step_inner(forward_step_func, data_iterator, model, optimizer, opt_param_scheduler, config)
    for mgr in _MEMORY_MANAGERS:
        mgr.end_step()
    if torch.cuda.is_available():
        from ..parallel import symm_mem
        if symm_mem.canaries_enabled():
            symm_mem.check_all_canaries()           # debugging aid: a write past a symmetric buffer stops the run here
    return out


def _train_step_inner(forward_step_func, data_iterator, model, optimizer, opt_param_scheduler, config=None):
    args = get_args()
    for m in model:
        m.zero_grad_buffer()
    optimizer.zero_grad()
    fb = get_forward_backward_func()
    fp8_recipe = None
    if getattr(args, "fp8_format", None):
        from ..models.te_compat import fp8_autocast, recipe_from_args
        fp8_recipe = recipe_from_args(args)
    import contextlib
    with (fp8_autocast(True, fp8_recipe) if fp8_recipe is not None else contextlib.nullcontext()):
        losses_reduced = fb(forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                            num_microbatches=get_num_microbatches(), seq_length=args.seq_length,
                            micro_batch_size=args.micro_batch_size, decoder_seq_length=None, forward_only=False)
    if getattr(args, "log_num_zeros_in_grad", False):
        # exact zeros in the reduced gradients, counted before the step consumes them (--log-num-zeros-in-grad)
        from ..patching.compat import count_zeros_fp32
        params = [p for m in model for p in m.parameters() if p.requires_grad]
        mpg = ps.get_model_parallel_group()
        zeros = count_zeros_fp32(params, mpg if dist.is_initialized() and dist.get_world_size(mpg) > 1 else None)
    ok, grad_norm, num_zeros = optimizer.step()
    if getattr(args, "log_num_zeros_in_grad", False):
        num_zeros = zeros
    if getattr(args, "balanced_moe_experts", False):
        # the experts that were busiest in this step are replicated on every expert-parallel rank for the next one
        from ..parallel.moe.moe_layer import MoELayer
        for chunk in model:
            for mod in chunk.modules():
                if isinstance(mod, MoELayer):
                    mod.refresh_hot_experts()
    if fp8_recipe is not None:
        from ..models.te_compat import clear_fp8_weight_cache
        clear_fp8_weight_cache()       # weights moved: cached quantised copies are stale
    if ok:
        opt_param_scheduler.step(1)
        skipped = 0
    else:
        skipped = 1
    loss_reduced = {}
    if losses_reduced:   # whichever rank holds a loss stage (the last rank; rank 0 for V-shaped schedules; both ends for bidirectional)
        for key in losses_reduced[0]:
            vals = [x[key] for x in losses_reduced]
            if torch.is_tensor(vals[0]) and vals[0].numel() == 2:
                t = torch.stack(vals).sum(0)
                loss_reduced[key] = t[0] / t[1]
            else:
                loss_reduced[key] = sum(vals) / len(vals)
    return loss_reduced, skipped, grad_norm, num_zeros


def training_log(loss_dict, iteration, elapsed, grad_norm, skipped, lr):
    args = get_args()
    bs = args.global_batch_size
    tokens = bs * args.seq_length
    world = args.world_size
    msg = f" iteration {iteration:8d}/{args.train_iters:8d} | elapsed time per iteration (ms): {elapsed * 1000:.1f}"
    msg += f" | learning rate: {lr:.3E} | global batch size: {bs:5d}"
    for k, v in loss_dict.items():
        msg += f" | {k}: {float(v):.6E}"
    if grad_norm is not None:
        msg += f" | grad norm: {float(grad_norm):.3f}"
    msg += f" | tokens/sec/GPU: {tokens / elapsed / world:.1f}"
    if args.op_cal_tflops or args.log_throughput:
        f = flops_mod.num_floating_point_operations(args, bs)
        hf = f + flops_mod.recompute_extra_flops(args, bs)
        peak = flops_mod.measured_peaks()["bf16_tflops"] * 1e12
        msg += f" | throughput per GPU (TFLOP/s/GPU): {f / elapsed / world / 1e12:.1f}"
        msg += f" | MFU: {f / elapsed / world / peak:.4f} | HFU: {hf / elapsed / world / peak:.4f}"
    print_rank_last(msg)


class ScalarWriter:
    """--tensorboard-dir: scalars go to a TensorBoard event file when the tensorboard package is importable, and always to
    ``scalars.jsonl`` in the same directory (one {"step", "tag", "value"} object per line)."""

    def __init__(self, log_dir, queue_size=1000, wandb_project="", wandb_name="", wandb_dir="", config=None):
        os.makedirs(log_dir, exist_ok=True)
        self.f = open(os.path.join(log_dir, "scalars.jsonl"), "a")
        try:
            from torch.utils.tensorboard import SummaryWriter
            self.tb = SummaryWriter(log_dir=log_dir, max_queue=queue_size)
        except Exception:
            self.tb = None
        self.wandb = None
        if wandb_project:                                  # --wandb-project: a third sink, when the package is installed
            try:
                import wandb
                wandb.init(project=wandb_project, name=wandb_name or None, dir=wandb_dir or log_dir, config=config or {})
                self.wandb = wandb
            except Exception:
                print_rank_last("note: --wandb-project given but the wandb package is not usable here; scalars go to "
                                f"{log_dir} only")

    def add_scalar(self, tag, value, step):
        self.f.write(json.dumps({"step": int(step), "tag": tag, "value": float(value)}) + "\n")
        self.f.flush()
        if self.tb is not None:
            self.tb.add_scalar(tag, float(value), int(step))
        if self.wandb is not None:
            self.wandb.log({tag: float(value)}, step=int(step))

    def close(self):
        self.f.close()
        if self.tb is not None:
            self.tb.close()
        if self.wandb is not None:
            self.wandb.finish()


def evaluate(forward_step_func, data_iterator, model, eval_iters):
    """Mean loss over ``eval_iters`` forward-only steps (reference: Megatron ``evaluate``; --eval-interval / --eval-iters)."""
    args = get_args()
    for m in model:
        m.eval()
    fb = get_forward_backward_func()
    totals = {}
    with torch.no_grad():
        for _ in range(eval_iters):
            losses = fb(forward_step_func=forward_step_func, data_iterator=data_iterator, model=model,
                        num_microbatches=get_num_microbatches(), seq_length=args.seq_length,
                        micro_batch_size=args.micro_batch_size, decoder_seq_length=None, forward_only=True)
            for d in losses or []:
                for k, v in d.items():
                    t = v.detach().float() if torch.is_tensor(v) else torch.tensor(float(v))
                    totals[k] = totals.get(k, 0) + t
    for m in model:
        m.train()
    out = {}
    for k, t in totals.items():
        out[k] = float(t[0] / t[1]) if (torch.is_tensor(t) and t.numel() == 2) else float(t) / max(1, eval_iters * get_num_microbatches())
    return out


def _moe_routers(model):
    from ..parallel.moe.router import TopKRouter
    return [m for chunk in model for m in chunk.modules() if isinstance(m, TopKRouter)]


def check_kernel_status():
    """Raise if a device-side bounded wait expired since the last check (GEMM mbarriers, all-gather / reduce-scatter
    flags, MoE, Ulysses, fused optimizer step): such a kernel returns early with its outputs not computed, so the step
    that contained it is invalid.  The RuntimeError names the wait's code and reaches the TTP exception handler.
    Call after the step's synchronize; costs one 4-byte read per device that has launched such kernels."""
    from ..ops import gemm as G
    G.check_status()


def _model_device(model) -> torch.device:
    """Device of the model's parameters (a chunk made of no-op layers only has none: any other chunk answers)."""
    return next((p.device for m in model for p in m.parameters()), torch.device("cpu"))


def calc_params_l2_norm(model) -> float:
    """L2 norm of all parameters of the job: tensor-parallel duplicates and shared embeddings counted once, summed over
    the model-parallel group (and the expert-parallel ranks for expert weights)."""
    dense = torch.zeros(1, dtype=torch.float32, device=_model_device(model))
    expert = torch.zeros_like(dense)
    tp_rank = ps.get_tensor_model_parallel_rank()
    for chunk in model:
        for p in chunk.parameters():
            if getattr(p, "shared", False) or (not getattr(p, "tensor_model_parallel", False) and getattr(p, "allreduce", True) and tp_rank != 0):
                continue
            sq = p.detach().float().pow(2).sum()
            if getattr(p, "allreduce", True):
                dense += sq
            else:
                expert += sq
    if dist.is_initialized():
        mpg = ps.get_model_parallel_group()
        if dist.get_world_size(mpg) > 1:
            dist.all_reduce(dense, group=mpg)
            dist.all_reduce(expert, group=mpg)
        if ps.get_expert_model_parallel_world_size() > 1:
            dist.all_reduce(expert, group=ps.get_expert_model_parallel_group())
    return float((dense + expert).sqrt())


def train(forward_step_func, model, optimizer, opt_param_scheduler, train_data_iterator, process_non_loss_data_func=None):
    args = get_args()
    for m in model:
        m.train()
    if getattr(args, "manual_gc", False):
        import gc
        gc.disable()                         # collections happen only where the loop asks for them
        gc.collect()
    iteration = args.iteration
    prof = None
    if args.profile and (args.profile_ranks == [-1] or args.rank in args.profile_ranks):
        from ..utils.profiler import build_profiler
        prof = build_profiler(args)
        prof.__enter__()
    history = []
    writer = None
    if args.tensorboard_dir and args.rank == args.world_size - 1:
        writer = ScalarWriter(args.tensorboard_dir, getattr(args, "tensorboard_queue_size", 1000), getattr(args, "wandb_project", ""),
                              getattr(args, "wandb_exp_name", ""), getattr(args, "wandb_save_dir", ""),
                              {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool))})
        if getattr(args, "log_world_size_to_tensorboard", False):
            writer.add_scalar("world-size", args.world_size, iteration)
    routers = _moe_routers(model) if (getattr(args, "print_expert_load", False) or getattr(args, "enable_expert_placement", False)) else []
    planners = {}
    while iteration < args.train_iters:
        t0 = time.time()
        loss_dict, skipped, grad_norm, num_zeros = train_step(forward_step_func, train_data_iterator, model, optimizer,
                                                              opt_param_scheduler)
        iteration += 1
        if getattr(args, "manual_gc", False) and args.manual_gc_interval and iteration % args.manual_gc_interval == 0:
            import gc
            gc.collect()                     # every rank at the same step: no rank stalls the others at a random moment
        if torch.cuda.is_available() and _model_device(model).type == "cuda":
            torch.cuda.synchronize()
        check_kernel_status()
        elapsed = time.time() - t0
        if prof is not None:
            prof.step()
        if iteration % args.log_interval == 0:
            if getattr(args, "log_num_zeros_in_grad", False) and num_zeros is not None:
                loss_dict["num zeros"] = float(num_zeros)
            if getattr(args, "log_params_norm", False):
                loss_dict["params norm"] = calc_params_l2_norm(model)
            if args.num_experts and args.moe_aux_loss_coeff > 0 and getattr(args, "moe_model_type", "") != "deepspeed_moe":
                # auxiliary losses the routers attached inside the model: mean over the MoE layers (and per layer with
                # --moe-per-layer-logging), averaged over the micro-batches and steps since the last log line
                from ..parallel.moe.moe_utils import reduce_moe_metrics
                calls = get_num_microbatches() * min(args.log_interval, iteration)
                tracker = ps.get_moe_layer_wise_logging_tracker()
                if "load_balancing_loss" not in tracker:         # a stage without MoE layers still joins the reduction
                    dev = _model_device(model)
                    tracker["load_balancing_loss"] = {"values": torch.zeros(args.num_layers, device=dev)}
                for name, per_layer in reduce_moe_metrics(tracker, calls).items():
                    n_moe = max(1, int((per_layer != 0).sum()))
                    loss_dict[name] = per_layer.sum() / n_moe
                    if getattr(args, "moe_per_layer_logging", False):
                        for i, x in enumerate(per_layer.tolist()):
                            if x != 0:
                                loss_dict[f"{name} layer {i + 1}"] = x
            training_log(loss_dict, iteration, elapsed, grad_norm, skipped, optimizer.param_groups[0]["lr"])
            if writer is not None and iteration % max(1, getattr(args, "tensorboard_log_interval", 1)) == 0:
                for k, v in loss_dict.items():
                    writer.add_scalar(k, float(v), iteration)
                if getattr(args, "log_learning_rate_to_tensorboard", True):
                    writer.add_scalar("learning-rate", optimizer.param_groups[0]["lr"], iteration)
                if getattr(args, "log_loss_scale_to_tensorboard", True) and hasattr(optimizer, "get_loss_scale"):
                    writer.add_scalar("loss-scale", float(optimizer.get_loss_scale()), iteration)
                if getattr(args, "log_timers_to_tensorboard", False):
                    writer.add_scalar("iteration-time", elapsed, iteration)
                    writer.add_scalar("tokens-per-second", args.global_batch_size * args.seq_length / elapsed, iteration)
                else:
                    writer.add_scalar("iteration-time", elapsed, iteration)
                if getattr(args, "log_memory_to_tensorboard", False) and torch.cuda.is_available():
                    writer.add_scalar("mem-allocated-bytes", torch.cuda.memory_allocated(), iteration)
                    writer.add_scalar("mem-max-allocated-bytes", torch.cuda.max_memory_allocated(), iteration)
                    writer.add_scalar("mem-reserved-bytes", torch.cuda.memory_reserved(), iteration)
                if grad_norm is not None:
                    writer.add_scalar("grad-norm", float(grad_norm), iteration)
        if routers and (iteration % args.log_interval == 0 or
                        (getattr(args, "enable_expert_placement", False) and iteration % args.expert_placement_freq == 0)):
            _expert_load_step(args, model, optimizer, routers, planners, iteration)
        if args.eval_interval and args.eval_iters and iteration % args.eval_interval == 0:
            ev = evaluate(forward_step_func, train_data_iterator, model, args.eval_iters)
            print_rank_last(f" validation at iteration {iteration:8d} | " + " | ".join(f"{k}: {v:.6E}" for k, v in ev.items()))
            if writer is not None:
                for k, v in ev.items():
                    writer.add_scalar(f"{k} validation", v, iteration)
                    if getattr(args, "log_validation_ppl_to_tensorboard", False) and "loss" in k:
                        writer.add_scalar(f"{k} validation ppl", math.exp(min(20.0, v)), iteration)
        history.append({k: float(v) for k, v in loss_dict.items()})
        if args.save and args.save_interval and iteration % args.save_interval == 0:
            from ..checkpointing import save_checkpoint
            save_checkpoint(iteration, model, optimizer, opt_param_scheduler)
        if args.exit_interval and iteration % args.exit_interval == 0:
            break
    if prof is not None:
        prof.__exit__(None, None, None)
    if writer is not None:
        writer.close()
    args.iteration = iteration
    return history


def _expert_load_step(args, model, optimizer, routers, planners, iteration):
    """--print-expert-load: log the tokens each expert received since the last report.  --enable-expert-placement: every
    --expert-placement-freq iterations feed the loads to a planner per MoE layer and move expert weights between the
    expert-parallel ranks when that lowers the heaviest rank's load (reference: mindspeed/core/transformer/moe/
    expert_placement/executor.py:44-586 and its hook in mindspeed/training.py:78-160)."""
    from ..parallel.moe.expert_placement import ExpertPlacementExecutor, ExpertPlacementPlanner
    ep = ps.get_expert_model_parallel_world_size()
    for li, r in enumerate(routers):
        load = r.pop_expert_load()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(load, group=ps.get_data_parallel_group(with_context_parallel=True))
        if getattr(args, "print_expert_load", False):
            print_rank_0(f" iteration {iteration:8d} | moe layer {li} tokens per expert: {[int(x) for x in load.tolist()]}")
        if getattr(args, "enable_expert_placement", False) and ep > 1 and iteration % args.expert_placement_freq == 0:
            # --enable-fine-grained-expert-placement: experts only move when the heaviest rank is more than the threshold
            # above the mean (reference: expert_placement/executor.py, fine_grained_expert_placement_thre)
            thr = args.fine_grained_expert_placement_thre if getattr(args, "enable_fine_grained_expert_placement", False) else None
            pl = planners.setdefault(li, ExpertPlacementPlanner(r.num_experts, ep, thr))
            pl.record(load)
            new = pl.plan()
            if new != pl.placement:
                layer = _moe_layer_of(model, r)
                tensors = [p.data for p in layer.experts.parameters()]
                ExpertPlacementExecutor(ps.get_expert_model_parallel_group()).apply(tensors, pl.placement, new)
                r.permute_experts(pl.placement, new)
                pl.commit(new)
                if hasattr(optimizer, "reload_model_params"):
                    optimizer.reload_model_params()


def _moe_layer_of(model, router):
    from ..parallel.moe.moe_layer import MoELayer
    for chunk in model:
        for m in chunk.modules():
            if isinstance(m, MoELayer) and m.router is router:
                return m
    raise RuntimeError("router does not belong to a MoE layer of this model")


def pretrain(train_valid_test_dataset_provider, model_provider, model_type=None, forward_step_func=None,
             process_non_loss_data_func=None, extra_args_provider=None, args_defaults=None, args_list=None):
    """Full entry: initialise, (optionally) run the auto-settings search and return, build, train, save."""
    args = initialize_megatron(extra_args_provider, args_defaults, args_list=args_list)
    if os.getenv("OOTB_OPTIMIZER_PARSE_ARGS", "FALSE") == "TRUE":
        # a search asks what this launch resolves to: write the validated arguments and stop
        from ..auto_settings.profiling_parse import dump_settings
        dump_settings(args, args.profile_save_path)
        print_rank_0("OOTB_OPTIMIZER_PARSE_ARGS: arguments written, exiting")
        return []
    if args.auto_settings:
        from ..auto_settings import AutoSettings
        return AutoSettings().auto_setting_fun(args)
    model, optimizer, sched = setup_model_and_optimizer(model_provider)
    if os.getenv("OOTB_OPTIMIZER_PARSE_MODEL", "FALSE") == "TRUE":
        from ..auto_settings.profiling_parse import dump_model_params
        if ps.get_data_parallel_rank() == 0 and ps.get_tensor_model_parallel_rank() == 0:
            dump_model_params(model, ps.get_pipeline_model_parallel_rank(), args.profile_save_path)
        print_rank_0("OOTB_OPTIMIZER_PARSE_MODEL: parameter tables written, exiting")
        return []
    if args.ttp_enabled:
        from ..checkpointing import load_fault_dump, save_fault_dump, wait_for_fault_dump
        from ..ttp import install_ttp

        def dump(ranks):
            # the controller names the ranks of one complete replica; each of them writes its shards without collectives
            if args.rank in ranks:
                save_fault_dump(args.iteration, model, optimizer, args.ttp_dump_dir, save_optimizer=args.ttp_save_optimizer,
                                save_rng=args.ttp_save_rng, keep=args.ttp_max_dump_ckpt_to_keep)
        install_ttp(args, dump_fn=dump)
        # a kernel that waits for a peer which has died must give up before the heartbeat declares this rank dead too
        from ..ops import fused_comm
        fused_comm.WAIT_LIMIT_MS = min(fused_comm.WAIT_LIMIT_MS, max(200, int(args.ttp_heartbeat_timeout_ms * 2 // 3)))
        if not args.load and os.path.isdir(args.ttp_dump_dir) and os.listdir(args.ttp_dump_dir):
            # restart after a fault: wait for the dump of this rank to be complete, then resume from it
            found = wait_for_fault_dump(args.ttp_dump_dir, [args.rank], timeout_s=args.ttp_wait_dump_file_timeout)
            if found is not None:
                args.iteration = load_fault_dump(model, optimizer if args.ttp_save_optimizer else None, found)
    train_iter = train_valid_test_dataset_provider(args)
    if getattr(args, "exit_on_missing_checkpoint", False) and args.load and not args.iteration:
        from ..checkpointing import read_latest_iteration
        if read_latest_iteration(args.load) is None:
            print_rank_0(f"--exit-on-missing-checkpoint: no checkpoint under {args.load}, exiting")
            return []
    if getattr(args, "skip_train", False):
        # --skip-train: no training steps; evaluate if asked to, then fall through to the final save
        history = []
        if args.eval_iters:
            ev = evaluate(forward_step_func, train_iter, model, args.eval_iters)
            print_rank_last(" validation loss (no training): " + " | ".join(f"{k}: {v:.6E}" for k, v in ev.items()))
            history.append({f"validation {k}": v for k, v in ev.items()})
    else:
        history = train(forward_step_func, model, optimizer, sched, train_iter, process_non_loss_data_func)
    if args.save:
        from ..checkpointing import finalize_async_save, save_checkpoint
        save_checkpoint(args.iteration, model, optimizer, sched)
        finalize_async_save(blocking=True)       # --async-save: the last checkpoint is on disk before pretrain returns
    return history
