"""Command-line arguments: Megatron-compatible core flags + every feature's flags.

Validation order is the reference's sandwich (mindspeed/core/megatron_basic/arguments_basic.py:37-61):
feature pre-validation -> core validation -> feature post-validation -> feature validation.
``core_transformer_config_from_args`` mirrors *every* flag onto the config object.
"""
from __future__ import annotations

import argparse
import dataclasses
import os

import torch
import torch.nn.functional as F

from ..config import MLATransformerConfig, TransformerConfig
from ..features import get_features_manager


def _core_args(p: argparse.ArgumentParser):
    g = p.add_argument_group("model")
    g.add_argument("--num-layers", type=int, default=None)
    g.add_argument("--hidden-size", type=int, default=None)
    g.add_argument("--ffn-hidden-size", type=int, default=None)
    g.add_argument("--num-attention-heads", type=int, default=None)
    g.add_argument("--kv-channels", type=int, default=None)
    g.add_argument("--group-query-attention", action="store_true")
    g.add_argument("--num-query-groups", type=int, default=None)
    g.add_argument("--max-position-embeddings", type=int, default=None)
    g.add_argument("--position-embedding-type", type=str, default="learned_absolute",
                   choices=["learned_absolute", "rope", "none", "alibi", "yarn"])
    g.add_argument("--use-rotary-position-embeddings", action="store_true")
    g.add_argument("--rotary-base", type=int, default=10000)
    g.add_argument("--rotary-percent", type=float, default=1.0)
    g.add_argument("--rotary-interleaved", action="store_true")
    g.add_argument("--rotary-seq-len-interpolation-factor", type=int, default=None)
    g.add_argument("--use-rope-scaling", action="store_true")
    g.add_argument("--normalization", type=str, default="LayerNorm", choices=["LayerNorm", "RMSNorm"])
    g.add_argument("--norm-epsilon", type=float, default=1e-5)
    g.add_argument("--apply-layernorm-1p", action="store_true")
    g.add_argument("--swiglu", action="store_true")
    g.add_argument("--squared-relu", action="store_true")
    g.add_argument("--disable-bias-linear", action="store_false", dest="add_bias_linear")
    g.add_argument("--add-qkv-bias", action="store_true")
    g.add_argument("--qk-layernorm", action="store_true")
    g.add_argument("--window-size", type=lambda t: tuple(int(x) for x in t.split(",")), default=None,
                   help="sliding-window attention: 'left,right' keys a query sees (-1 = unbounded)")
    g.add_argument("--untie-embeddings-and-output-weights", action="store_true")
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128)
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--padded-vocab-size", type=int, default=None)
    g.add_argument("--hidden-dropout", type=float, default=0.1)
    g.add_argument("--attention-dropout", type=float, default=0.1)
    g.add_argument("--init-method-std", type=float, default=0.02)
    g.add_argument("--apply-query-key-layer-scaling", action="store_true")
    g.add_argument("--attention-softmax-in-fp32", action="store_true")
    g.add_argument("--use-flash-attn", action="store_true")
    g.add_argument("--mtp-num-layers", type=int, default=None)
    g.add_argument("--mtp-loss-scaling-factor", type=float, default=0.1)

    g = p.add_argument_group("moe")
    g.add_argument("--num-experts", type=int, default=None)
    g.add_argument("--moe-router-topk", type=int, default=2)
    g.add_argument("--moe-hierarchical-alltoallv", action="store_true")
    g.add_argument("--no-create-attention-mask-in-dataloader", action="store_false", dest="create_attention_mask_in_dataloader")
    g.add_argument("--overlap-param-gather-with-optimizer-step", action="store_true")
    g.add_argument("--moe-router-dtype", type=str, default=None, choices=[None, "fp32", "fp64"],
                   help="precision of the router's logits, softmax and top-k (fp32 when unset)")
    g.add_argument("--seq-aux", action="store_true", help="the same as --moe-router-load-balancing-type seq_aux_loss")
    g.add_argument("--moe-router-load-balancing-type", type=str, default="aux_loss",
                   choices=["aux_loss", "seq_aux_loss", "sinkhorn", "none"])
    g.add_argument("--moe-router-score-function", type=str, default="softmax", choices=["softmax", "sigmoid"])
    g.add_argument("--moe-router-pre-softmax", action="store_true")
    g.add_argument("--moe-router-topk-scaling-factor", type=float, default=None)
    g.add_argument("--moe-router-enable-expert-bias", action="store_true")
    g.add_argument("--moe-router-bias-update-rate", type=float, default=1e-3)
    g.add_argument("--moe-router-num-groups", type=int, default=None)
    g.add_argument("--moe-router-group-topk", type=int, default=None)
    g.add_argument("--moe-aux-loss-coeff", type=float, default=0.0)
    g.add_argument("--moe-z-loss-coeff", type=float, default=None)
    g.add_argument("--moe-input-jitter-eps", type=float, default=None)
    g.add_argument("--moe-token-dispatcher-type", type=str, default="allgather",
                   choices=["allgather", "alltoall", "alltoall_seq", "flex"])
    g.add_argument("--moe-grouped-gemm", action="store_true")
    g.add_argument("--moe-ffn-hidden-size", type=int, default=None)
    g.add_argument("--moe-shared-expert-intermediate-size", type=int, default=None)
    g.add_argument("--moe-shared-expert-overlap", action="store_true")
    g.add_argument("--moe-layer-freq", type=str, default="1")
    g.add_argument("--moe-expert-capacity-factor", type=float, default=None)
    g.add_argument("--moe-pad-expert-input-to-capacity", action="store_true")
    g.add_argument("--moe-token-drop-policy", type=str, default="probs", choices=["probs", "position"])
    g.add_argument("--moe-layer-recompute", action="store_true")
    g.add_argument("--moe-permute-fusion", action="store_true")
    g.add_argument("--moe-per-layer-logging", action="store_true")
    g.add_argument("--first-k-dense-replace", type=int, default=0)

    g = p.add_argument_group("parallel")
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--num-layers-per-virtual-pipeline-stage", type=int, default=None)
    g.add_argument("--num-virtual-stages-per-pipeline-rank", type=int, default=None)
    g.add_argument("--context-parallel-size", type=int, default=1)
    g.add_argument("--expert-model-parallel-size", type=int, default=1)
    g.add_argument("--expert-tensor-parallel-size", type=int, default=None)
    g.add_argument("--sequence-parallel", action="store_true")
    g.add_argument("--use-distributed-optimizer", action="store_true")
    g.add_argument("--num-distributed-optimizer-instances", type=int, default=1)
    g.add_argument("--overlap-grad-reduce", action="store_true")
    g.add_argument("--overlap-param-gather", action="store_true")
    g.add_argument("--ddp-bucket-size", type=int, default=None)
    g.add_argument("--ddp-average-in-collective", action="store_true")
    g.add_argument("--no-gradient-accumulation-fusion", action="store_false", dest="gradient_accumulation_fusion")
    g.add_argument("--accumulate-allreduce-grads-in-fp32", action="store_true")
    g.add_argument("--distributed-backend", type=str, default="nccl", choices=["nccl", "gloo"])
    g.add_argument("--distributed-timeout-minutes", type=int, default=10)
    g.add_argument("--use-tp-pp-dp-mapping", action="store_true")
    g.add_argument("--variable-seq-lengths", action="store_true")
    g.add_argument("--overlap-p2p-communication", action="store_true", dest="overlap_p2p_comm")
    g.add_argument("--decoder-first-pipeline-num-layers", type=int, default=None)
    g.add_argument("--decoder-last-pipeline-num-layers", type=int, default=None)
    g.add_argument("--nccl-communicator-config-path", type=str, default=None)
    g.add_argument("--local-rank", "--local_rank", type=int, default=None)

    g = p.add_argument_group("training")
    g.add_argument("--micro-batch-size", type=int, default=1)
    g.add_argument("--global-batch-size", type=int, default=None)
    g.add_argument("--seq-length", type=int, default=None)
    g.add_argument("--train-iters", type=int, default=None)
    g.add_argument("--eval-iters", type=int, default=0)
    g.add_argument("--eval-interval", type=int, default=1000)
    g.add_argument("--log-interval", type=int, default=1)
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--bf16", action="store_true")
    g.add_argument("--fp16", action="store_true")
    g.add_argument("--loss-scale", type=float, default=None)
    g.add_argument("--initial-loss-scale", type=float, default=2 ** 32)
    g.add_argument("--optimizer", type=str, default="adam", choices=["adam", "sgd", "muon"])
    g.add_argument("--lr", type=float, default=None)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", type=str, default="constant", choices=["constant", "linear", "cosine", "inverse-square-root", "WSD"])
    g.add_argument("--lr-decay-iters", type=int, default=None)
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--lr-warmup-fraction", type=float, default=None)
    g.add_argument("--weight-decay", type=float, default=0.01)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.999)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--clip-grad", type=float, default=1.0)
    g.add_argument("--recompute-granularity", type=str, default=None, choices=[None, "full", "selective"])
    g.add_argument("--recompute-method", type=str, default=None, choices=[None, "uniform", "block"])
    g.add_argument("--recompute-num-layers", type=int, default=None)
    g.add_argument("--recompute-activations", action="store_true")
    g.add_argument("--distribute-saved-activations", action="store_true")
    g.add_argument("--calculate-per-token-loss", action="store_true")
    g.add_argument("--use-cpu-initialization", action="store_true")
    g.add_argument("--check-for-nan-in-loss-and-grad", action="store_true")
    g.add_argument("--exit-interval", type=int, default=None)
    g.add_argument("--transformer-impl", type=str, default="local", choices=["local", "transformer_engine"])
    g.add_argument("--use-mcore-models", action="store_true")
    g.add_argument("--no-masked-softmax-fusion", action="store_false", dest="masked_softmax_fusion")
    g.add_argument("--no-bias-dropout-fusion", action="store_false", dest="bias_dropout_fusion")
    g.add_argument("--no-bias-swiglu-fusion", action="store_false", dest="bias_swiglu_fusion")
    g.add_argument("--yaml-cfg", type=str, default=None)
    # --- further Megatron training flags that launch scripts of the reference pass ---
    g.add_argument("--train-samples", type=int, default=None, help="length of training in samples (instead of --train-iters)")
    g.add_argument("--skip-train", action="store_true", help="build, load and evaluate / save without training steps")
    g.add_argument("--start-weight-decay", type=float, default=None)
    g.add_argument("--end-weight-decay", type=float, default=None)
    g.add_argument("--weight-decay-incr-style", type=str, default="constant", choices=["constant", "linear", "cosine"])
    g.add_argument("--log-num-zeros-in-grad", action="store_true")
    g.add_argument("--log-params-norm", action="store_true")
    g.add_argument("--manual-gc", action="store_true", help="collect garbage only every --manual-gc-interval steps, on all ranks at once")
    g.add_argument("--manual-gc-interval", type=int, default=0)
    g.add_argument("--timing-log-level", type=int, default=0, choices=[0, 1, 2])
    g.add_argument("--timing-log-option", type=str, default="minmax", choices=["max", "minmax", "all"])
    g.add_argument("--no-barrier-with-level-1-timing", action="store_false", dest="barrier_with_L1_time")
    g.add_argument("--no-bias-gelu-fusion", action="store_false", dest="bias_gelu_fusion")
    g.add_argument("--no-rope-fusion", action="store_false", dest="apply_rope_fusion")
    g.add_argument("--no-position-embedding", action="store_false", dest="add_position_embedding")
    g.add_argument("--use-legacy-models", action="store_true")
    g.add_argument("--spec", type=str, nargs="*", default=None)
    g.add_argument("--use-torch-fsdp2", action="store_true", help="parameters sharded over data-parallel ranks (the --layerzero path)")
    g.add_argument("--use-custom-fsdp", action="store_true", help="with --data-parallel-sharding-strategy: the --layerzero path")
    g.add_argument("--data-parallel-sharding-strategy", type=str, default="no_shard",
                   choices=["no_shard", "optim", "optim_grads", "optim_grads_params"])
    g.add_argument("--fp8-amax-history-len", type=int, default=1024)
    g.add_argument("--fp8-amax-compute-algo", type=str, default="max", choices=["max", "most_recent"])
    g.add_argument("--short-seq-prob", type=float, default=0.1)
    g.add_argument("--img-h", type=int, default=224)
    g.add_argument("--img-w", type=int, default=224)
    g.add_argument("--patch-dim", type=int, default=16)

    g = p.add_argument_group("data / checkpoint")
    g.add_argument("--data-path", nargs="*", default=None)
    g.add_argument("--mock-data", action="store_true")
    g.add_argument("--split", type=str, default="100,0,0")
    g.add_argument("--tokenizer-type", type=str, default="NullTokenizer")
    g.add_argument("--tokenizer-model", type=str, default=None)
    g.add_argument("--vocab-file", type=str, default=None, help="GPT2BPETokenizer: vocab.json")
    g.add_argument("--merge-file", type=str, default=None, help="GPT2BPETokenizer: merges.txt")
    g.add_argument("--auto-detect-ckpt-format", action="store_true")
    g.add_argument("--dist-ckpt-format", type=str, default="torch_dist", choices=["torch_dist"])
    g.add_argument("--exit-on-missing-checkpoint", action="store_true",
                   help="stop when --load is given and holds no checkpoint (instead of starting from scratch)")
    g.add_argument("--use-checkpoint-opt_param-scheduler", "--use-checkpoint-opt-param-scheduler", action="store_true",
                   dest="use_checkpoint_opt_param_scheduler", help="take the schedule's settings from the checkpoint")
    g.add_argument("--no-shared-storage", action="store_false", dest="shared_storage")
    g.add_argument("--save", type=str, default=None)
    g.add_argument("--load", type=str, default=None)
    g.add_argument("--save-interval", type=int, default=None)
    g.add_argument("--no-save-optim", action="store_true")
    g.add_argument("--no-save-rng", action="store_true")
    g.add_argument("--no-load-optim", action="store_true")
    g.add_argument("--no-load-rng", action="store_true")
    g.add_argument("--finetune", action="store_true",
                   help="load the model weights only (no optimizer, scheduler or RNG state) and start counting iterations at 0")
    g.add_argument("--ckpt-format", type=str, default="torch_dist", choices=["torch", "torch_dist"])
    g.add_argument("--use-dist-ckpt", action="store_true")
    g.add_argument("--async-save", action="store_true")
    g.add_argument("--ckpt-fully-parallel-save", action="store_true")
    g.add_argument("--dist-ckpt-optim-sharding-type", type=str, default="fully_sharded_bucket_space",
                   choices=["fully_sharded_bucket_space", "dp_zero_gather_scatter", "fully_sharded_model_space"])
    g.add_argument("--tensorboard-dir", type=str, default=None)
    g.add_argument("--tensorboard-log-interval", type=int, default=1, help="write scalars every this many iterations")
    g.add_argument("--tensorboard-queue-size", type=int, default=1000)
    g.add_argument("--log-timers-to-tensorboard", action="store_true")
    g.add_argument("--log-memory-to-tensorboard", action="store_true")
    g.add_argument("--log-world-size-to-tensorboard", action="store_true")
    g.add_argument("--log-validation-ppl-to-tensorboard", action="store_true")
    g.add_argument("--no-log-learnig-rate-to-tensorboard", "--no-log-learning-rate-to-tensorboard", action="store_false",
                   dest="log_learning_rate_to_tensorboard")
    g.add_argument("--no-log-loss-scale-to-tensorboard", action="store_false", dest="log_loss_scale_to_tensorboard")
    g.add_argument("--wandb-project", type=str, default="", help="also send the scalars to Weights & Biases (when the package exists)")
    g.add_argument("--wandb-exp-name", type=str, default="")
    g.add_argument("--wandb-save-dir", type=str, default="")
    g.add_argument("--log-throughput", action="store_true")
    g.add_argument("--num-workers", type=int, default=0)
    g.add_argument("--reset-position-ids", action="store_true")
    g.add_argument("--eod-mask-loss", action="store_true")
    return p


def build_parser(extra_args_provider=None) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="mindspeed_b200 arguments", allow_abbrev=False)
    _core_args(p)
    get_features_manager().register_features_args(p)
    if extra_args_provider is not None:
        p = extra_args_provider(p) or p
    return p


def parse_args(extra_args_provider=None, ignore_unknown_args=False, args_list=None):
    p = build_parser(extra_args_provider)
    if ignore_unknown_args:
        args, _ = p.parse_known_args(args_list)
    else:
        args = p.parse_args(args_list)
    if args.yaml_cfg:
        from .yaml_arguments import load_yaml
        args = load_yaml(args.yaml_cfg, args)
    args._parser = p                       # validate_args compares values with the parser's defaults (features/flag_policy.py)
    args.rank = int(os.getenv("RANK", "0"))
    args.world_size = int(os.getenv("WORLD_SIZE", "1"))
    if args.local_rank is None:
        args.local_rank = int(os.getenv("LOCAL_RANK", "0"))
    return args


def _layer_pattern(text: str):
    """``--moe-layer-freq``: an integer N (every N-th layer) or a list expression such as ``([0]*3+[1]*1)*4`` - lists of
    integers joined by ``+`` and repeated by ``*``.  Evaluated from the syntax tree: nothing but those forms is accepted."""
    import ast

    def ev(n):
        if isinstance(n, ast.Expression):
            return ev(n.body)
        if isinstance(n, ast.Constant) and isinstance(n.value, int):
            return n.value
        if isinstance(n, (ast.List, ast.Tuple)):
            return [ev(e) for e in n.elts]
        if isinstance(n, ast.BinOp) and isinstance(n.op, (ast.Add, ast.Mult)):
            a, b = ev(n.left), ev(n.right)
            if isinstance(n.op, ast.Add) and isinstance(a, list) and isinstance(b, list):
                return a + b
            if isinstance(n.op, ast.Mult) and (isinstance(a, list) != isinstance(b, list) or (isinstance(a, int) and isinstance(b, int))):
                return a * b
        raise AssertionError(f"--moe-layer-freq: cannot read {text!r} (an integer, or integer lists combined with + and *)")
    return ev(ast.parse(text.strip(), mode="eval"))


def _core_validate(args):
    mp = args.tensor_model_parallel_size * args.pipeline_model_parallel_size * args.context_parallel_size
    if args.world_size % mp != 0:
        raise AssertionError(f"world size {args.world_size} is not divisible by tp*pp*cp = {mp}")
    args.data_parallel_size = args.world_size // mp
    if args.global_batch_size is None:
        per_rank = sum(args.micro_batch_sizes) if getattr(args, "micro_batch_sizes", None) else args.micro_batch_size
        args.global_batch_size = per_rank * args.data_parallel_size
    if not getattr(args, "micro_batch_sizes", None) and args.global_batch_size % (args.micro_batch_size * args.data_parallel_size) != 0:
        raise AssertionError("global batch size must be divisible by micro batch size * data parallel size")
    if args.num_layers is None or args.hidden_size is None or args.num_attention_heads is None:
        raise AssertionError("--num-layers, --hidden-size and --num-attention-heads are required")
    if args.seq_length is None:
        raise AssertionError("--seq-length is required")
    if args.max_position_embeddings is None:
        args.max_position_embeddings = args.seq_length
    if args.ffn_hidden_size is None:
        args.ffn_hidden_size = int((4 * args.hidden_size * 2 / 3) / 64) * 64 if args.swiglu else 4 * args.hidden_size
    if args.kv_channels is None:
        args.kv_channels = args.hidden_size // args.num_attention_heads
    if not args.group_query_attention:
        args.num_query_groups = args.num_attention_heads
    elif args.num_query_groups is None:
        raise AssertionError("--group-query-attention needs --num-query-groups")
    if args.use_rotary_position_embeddings:
        args.position_embedding_type = "rope"
    if getattr(args, "seq_aux", False):
        args.moe_router_load_balancing_type = "seq_aux_loss"
    if not args.add_position_embedding and args.position_embedding_type == "learned_absolute":
        args.position_embedding_type = "none"                     # --no-position-embedding
    if args.train_samples is not None:
        if args.train_iters is not None:
            raise AssertionError("give --train-iters or --train-samples, not both")
        args.train_iters = args.train_samples // args.global_batch_size
    if args.start_weight_decay is None:
        args.start_weight_decay = args.end_weight_decay = args.weight_decay
    elif args.end_weight_decay is None:
        raise AssertionError("--start-weight-decay needs --end-weight-decay")
    elif args.weight_decay_incr_style == "constant" and args.start_weight_decay != args.end_weight_decay:
        raise AssertionError("--weight-decay-incr-style constant needs equal start and end weight decay")
    else:
        args.weight_decay = args.start_weight_decay
    if args.use_torch_fsdp2 or (args.use_custom_fsdp and args.data_parallel_sharding_strategy == "optim_grads_params"):
        args.layerzero = True                                        # parameters, gradients and optimizer state sharded
        args.use_distributed_optimizer = False                       # ... which includes what the distributed optimizer shards
    elif args.use_custom_fsdp and args.data_parallel_sharding_strategy in ("optim", "optim_grads"):
        args.use_distributed_optimizer = True                        # optimizer state (and reduce-scattered gradients) sharded
    if args.manual_gc and args.manual_gc_interval < 0:
        raise AssertionError("--manual-gc-interval must not be negative")
    args.params_dtype = torch.bfloat16 if args.bf16 else torch.float16 if args.fp16 else torch.float32
    if args.bf16:
        args.accumulate_allreduce_grads_in_fp32 = True
    if getattr(args, "reset_attention_mask", False):
        # packed documents: each attends to itself only; documents are concatenated along the sequence of one sample
        # --fix-sub-seq-length L replaces the documents' own boundaries by sub-sequences of L tokens (the last takes the
        # rest): every row of a batch then has the same boundaries, so any micro-batch size and synthetic data work
        fixed = 0 < (getattr(args, "fix_sub_seq_length", None) or -1) <= args.seq_length
        if args.micro_batch_size != 1 and not fixed:
            raise AssertionError("--reset-attention-mask takes --micro-batch-size 1 (packed documents share one sequence)")
        if getattr(args, "context_parallel_size", 1) > 1:
            raise AssertionError("--reset-attention-mask is not combined with context parallelism")
        if not getattr(args, "data_path", None) and not fixed:
            raise AssertionError("--reset-attention-mask needs --data-path: synthetic data has no document boundaries")
    if args.sequence_parallel and args.tensor_model_parallel_size == 1:
        args.sequence_parallel = False
    if args.recompute_activations:
        args.recompute_granularity = "selective"
    if args.padded_vocab_size is None and args.vocab_size is not None:
        mult = args.make_vocab_size_divisible_by * args.tensor_model_parallel_size
        args.padded_vocab_size = ((args.vocab_size + mult - 1) // mult) * mult
    vpp = None
    if args.num_layers_per_virtual_pipeline_stage is not None:
        per = args.num_layers // args.pipeline_model_parallel_size
        if per % args.num_layers_per_virtual_pipeline_stage != 0:
            raise AssertionError("layers per stage must be divisible by layers per virtual stage")
        vpp = per // args.num_layers_per_virtual_pipeline_stage
    elif args.num_virtual_stages_per_pipeline_rank is not None:
        vpp = args.num_virtual_stages_per_pipeline_rank
    args.virtual_pipeline_model_parallel_size = vpp
    if isinstance(args.moe_layer_freq, str):
        args.moe_layer_freq = _layer_pattern(args.moe_layer_freq)
    if args.num_experts is not None and args.expert_model_parallel_size > 1:
        if args.num_experts % args.expert_model_parallel_size != 0:
            raise AssertionError("num_experts must be divisible by expert parallel size")
    if args.ckpt_format == "torch_dist":
        args.use_dist_ckpt = True
    if getattr(args, "moe_use_sinkhorn", False):
        args.moe_router_load_balancing_type = "sinkhorn"
    n_shared = getattr(args, "n_shared_experts", None)
    if n_shared and not args.moe_shared_expert_intermediate_size:
        # DeepSeek-style count of always-on experts -> one shared MLP of n x the routed experts' width
        args.moe_shared_expert_intermediate_size = n_shared * (args.moe_ffn_hidden_size or args.ffn_hidden_size)
    cf = getattr(args, "moe_train_capacity_factor", None)
    if args.num_experts and cf is not None and cf != 1.0 and not getattr(args, "moe_no_drop", False):
        if getattr(args, "moe_expert_capacity_factor", None) is None:
            args.moe_expert_capacity_factor = cf                                    # legacy spelling of the capacity factor
    if getattr(args, "moe_no_drop", False):
        args.moe_expert_capacity_factor = None                                      # never drop tokens
    return args


def validate_args(args):
    fm = get_features_manager()
    fm.pre_validate_features_args(args)
    _core_validate(args)
    fm.post_validate_features_args(args)
    fm.validate_features_args(args)
    parser = getattr(args, "_parser", None)
    if parser is not None:
        from ..features.flag_policy import check_flags
        check_flags(args, parser)
    return args


def core_transformer_config_from_args(args, config_class=None) -> TransformerConfig:
    config_class = config_class or (MLATransformerConfig if getattr(args, "multi_head_latent_attention", False) else TransformerConfig)
    kw = {}
    for f in dataclasses.fields(config_class):
        if hasattr(args, f.name):
            kw[f.name] = getattr(args, f.name)
    kw["layernorm_epsilon"] = args.norm_epsilon
    kw["layernorm_zero_centered_gamma"] = args.apply_layernorm_1p
    kw["num_moe_experts"] = args.num_experts
    kw["first_pipeline_num_layers"] = args.decoder_first_pipeline_num_layers
    kw["last_pipeline_num_layers"] = args.decoder_last_pipeline_num_layers
    kw["pipeline_dtype"] = args.params_dtype
    kw["deallocate_pipeline_outputs"] = False
    kw["multi_latent_attention"] = bool(getattr(args, "multi_head_latent_attention", False))
    if args.swiglu:
        kw["activation_func"] = F.silu
        kw["gated_linear_unit"] = True
    elif args.squared_relu:
        kw["activation_func"] = lambda x: torch.pow(F.relu(x), 2)
    kw["bias_activation_fusion"] = False
    if getattr(args, "multi_head_latent_attention", False):
        kw.update(q_lora_rank=args.q_lora_rank, kv_lora_rank=args.kv_lora_rank, qk_head_dim=args.qk_nope_head_dim,
                  qk_pos_emb_head_dim=args.qk_rope_head_dim, v_head_dim=args.v_head_dim,
                  rope_type="yarn" if args.rope_scaling_type == "yarn" else "rope", rotary_base=args.rotary_base,
                  rotary_scaling_factor=args.rope_scaling_factor,
                  original_max_position_embeddings=args.rope_scaling_original_max_position_embeddings,
                  beta_fast=args.rope_scaling_beta_fast, beta_slow=args.rope_scaling_beta_slow,
                  mscale=args.rope_scaling_mscale, mscale_all_dim=args.rope_scaling_mscale_all_dim,
                  max_position_embeddings=args.max_position_embeddings)
    cfg = config_class(**kw)
    cfg.update_from_args(args)
    return cfg
