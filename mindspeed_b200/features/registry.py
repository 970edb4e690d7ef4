"""All feature classes, in application order (reference: mindspeed/features_manager/__init__.py:377-409).

Every class owns its flags.  Flag names are the reference's (including its historical spellings such
as ``--pre-tockens``) so launch scripts carry over; vendor-specific names that users already have in
scripts (``--use-ascend-mc2``, ``--use-ascend-coc``, ``--hccl-*``) are kept as aliases of the
hardware-neutral ones (``--use-fused-tp-comm``, ``--use-chunked-tp-comm``, ``--nccl-*``).
"""
from __future__ import annotations

from .feature import Feature, add_arg


# ======================================================================================
# level-0 basics
# ======================================================================================
class RequirementsBasicFeature(Feature):
    def __init__(self):
        super().__init__("requirements-basic", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--optimization-level", type=int, choices=[0, 1, 2], default=2,
                help="0: library GEMM + NCCL paths; 1: + fused single-GPU kernels; 2: + fused compute/communication kernels")
        add_arg(g, "--optimizer-selection", type=str, default="fused_adamw",
                choices=["fused_adamw", "fused_torch_adamw", "fused_ema_adamw"])
        add_arg(g, "--ai-framework", type=str, default="pytorch", choices=["pytorch", "mindspore"])

    def validate_args(self, args):
        if args.ai_framework != "pytorch":
            raise AssertionError("only the pytorch framework layer exists in this build")


class MegatronBasicFeature(Feature):
    def __init__(self):
        super().__init__("megatron-basic", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--use-fused-rmsnorm", action="store_true")
        add_arg(g, "--use-fused-swiglu", action="store_true")
        add_arg(g, "--use-fused-rotary-pos-emb", action="store_true")
        add_arg(g, "--use-fused-moe-token-permute-and-unpermute", action="store_true")
        add_arg(g, "--use-fused-ring-attention-update", action="store_true")
        add_arg(g, "--gemm-gradient-accumulation-fusion", action="store_true")

    def post_validate_args(self, args):
        if args.optimization_level >= 1:
            for k in ("use_fused_rmsnorm", "use_fused_swiglu", "use_fused_rotary_pos_emb",
                      "use_fused_moe_token_permute_and_unpermute"):
                setattr(args, k, True)


class TransformerEngineBasicFeature(Feature):
    """fp8 recipes and the TE-compatible module options
    (reference: mindspeed/features_manager/megatron_basic/transformer_engine_basic.py:41-272)."""

    def __init__(self):
        super().__init__("transformer-engine-basic", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--fp8-format", type=str, default=None, choices=["e4m3", "hybrid", "hif8"])
        add_arg(g, "--fp8-recipe", type=str, default="delayed",
                choices=["delayed", "tensorwise", "mxfp8", "mxfp8-32x32", "blockwise"])
        add_arg(g, "--no-use-gmm-fp8", action="store_false", dest="use_gmm_fp8")
        add_arg(g, "--te-comparison-with-cpu", action="store_true")
        add_arg(g, "--te-comparison-with-bf16", action="store_true")
        add_arg(g, "--te-gmm-mode", type=str, default="performance", choices=["performance", "compatible"])
        add_arg(g, "--fp8-reuse-quantized-weight", action="store_true")
        add_arg(g, "--qat-scheme", type=str, default=None, choices=[None, "w4a16", "w8a16", "w4a4"])
        add_arg(g, "--qat-quant-block-size", type=int, default=128)
        add_arg(g, "--qad-enable", action="store_true", default=False)
        add_arg(g, "--no-qad-enable", action="store_false", dest="qad_enable")
        add_arg(g, "--qad-teacher-load", type=str, default="")
        add_arg(g, "--kl-temperature", type=float, default=1.0)
        add_arg(g, "--kl-loss-weight", type=float, default=1.0)
        add_arg(g, "--kl-loss-reduction", type=str, default="mean", choices=["mean", "sum"])

    def validate_args(self, args):
        if args.fp8_format == "hif8":
            raise AssertionError("hif8 is an Ascend number format with no Blackwell tensor-core mode; use e4m3/hybrid")
        if args.fp8_format and args.fp8_recipe == "delayed" and getattr(args, "moe_grouped_gemm", False):
            pass


class QADFeature(Feature):
    """Quantisation-aware distillation (reference: mindspeed/features_manager/qad/qad_quant_engine.py:17-175)."""

    def __init__(self):
        super().__init__("qad-enable", optimization_level=0)

    def is_need_apply(self, args) -> bool:
        return bool(getattr(args, "qad_enable", False))

    def validate_args(self, args):
        if not args.qad_teacher_load:
            raise AssertionError("--qad-enable needs --qad-teacher-load (the teacher's checkpoint directory)")
        if args.kl_temperature <= 0:
            raise AssertionError(f"--kl-temperature must be positive, got {args.kl_temperature}")
        if args.kl_loss_weight < 0:
            raise AssertionError(f"--kl-loss-weight must not be negative, got {args.kl_loss_weight}")
        if getattr(args, "num_experts", None):
            raise AssertionError("--qad-enable covers dense models only (--num-experts is set)")
        if args.pipeline_model_parallel_size > 1:
            raise AssertionError("--qad-enable needs --pipeline-model-parallel-size 1: the loss compares the teacher's and "
                                 "the student's logits of one micro-batch on one rank")
        if getattr(args, "context_parallel_size", 1) > 1:
            raise AssertionError("--qad-enable is not combined with context parallelism")


class LegacySpellingsFeature(Feature):
    """Older spellings of current features and stored policies of the automated pipeline (reference: mindspeed/arguments.py:
    27-976, the argument groups that predate the feature classes).  ``pre_validate_args`` rewrites them onto the flags
    the framework reads, so both spellings run the same code."""

    def __init__(self):
        super().__init__("legacy-spellings", optimization_level=0)
        self.default_patches = True

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--use-nd-matmul", action="store_true", help="older name of --tp-2d")
        add_arg(g, "--nd1-dim1-size", type=int, default=1, help="with --use-nd-matmul: --tp-x")
        add_arg(g, "--nd2-dim1-size", type=int, default=1, help="with --use-nd-matmul: --tp-y")
        add_arg(g, "--optimize-vpp-send-recv-comm", action="store_true",
                help="--optimize-send-recv-comm for the interleaved schedule (one switch covers both here)")
        add_arg(g, "--enable-zero3", action="store_true", help="parameters, gradients and optimizer state sharded over "
                "the data-parallel group: the same as --layerzero")
        add_arg(g, "--shape-order", type=str, default="SBH", choices=["SBH", "BSH", "BSND", "BNSD"])
        add_arg(g, "--yarn-scaling-factor", type=float, default=1.0, help="older name of --rope-scaling-factor with yarn")
        add_arg(g, "--add-dense-bias", action="store_true", help="bias on the attention output projection even with --disable-bias-linear")
        add_arg(g, "--skip-bias-add", action="store_false", default=True)
        add_arg(g, "--additional-config", type=str, default=None,
                help="JSON / YAML file of {argument name: value} applied on top of the command line")
        add_arg(g, "--save-memory-ratio", type=float, default=0.20,
                help="--automated-pipeline: fraction of device memory the plan must leave free")
        add_arg(g, "--optimized-mbs-list", type=str, default=None)
        add_arg(g, "--mbs-idx", type=int, default=None)
        add_arg(g, "--pp-schedule-list", type=str, default=None)
        add_arg(g, "--optimized-mbs-mode", action="store_false")

    def pre_validate_args(self, args):
        if args.additional_config:
            import json
            with open(args.additional_config) as f:
                txt = f.read()
            try:
                extra = json.loads(txt)
            except ValueError:
                import yaml
                extra = yaml.safe_load(txt)
            if not isinstance(extra, dict):
                raise AssertionError("--additional-config must hold a mapping of argument names to values")
            for k, v in extra.items():
                k = k.lstrip("-").replace("-", "_")
                if not hasattr(args, k):
                    raise AssertionError(f"--additional-config: unknown argument {k!r}")
                setattr(args, k, v)
        if args.use_nd_matmul:
            if args.tp_2d:
                raise AssertionError("--use-nd-matmul is the older name of --tp-2d; give one of them")
            tp = args.tensor_model_parallel_size
            if tp % args.nd1_dim1_size or tp % args.nd2_dim1_size:
                raise AssertionError("tensor_model_parallel_size must be divisible by nd1_dim1_size and by nd2_dim1_size")
            if args.nd1_dim1_size * args.nd2_dim1_size != tp:
                raise AssertionError("--nd1-dim1-size x --nd2-dim1-size must equal --tensor-model-parallel-size (the x and y "
                                     "extents of the 2-D tensor-parallel grid)")
            args.tp_2d, args.tp_x, args.tp_y = True, args.nd1_dim1_size, args.nd2_dim1_size
        if args.optimize_vpp_send_recv_comm:
            args.optimize_send_recv_comm = True
        if args.enable_zero3:
            args.layerzero = True
        if args.yarn_scaling_factor != 1.0 and getattr(args, "rope_scaling_factor", 1.0) == 1.0:
            args.rope_scaling_factor = args.yarn_scaling_factor
        args.micro_batch_sizes = None
        if args.optimized_mbs_list and args.optimized_mbs_mode:
            import ast
            v = args.optimized_mbs_list
            sizes = list(ast.literal_eval(v if v.strip().startswith("[") else f"[{v}]")) if isinstance(v, str) else list(v)
            if not sizes or any((not isinstance(b, int)) or b < 1 for b in sizes):
                raise AssertionError("--optimized-mbs-list is a list of positive micro-batch sizes, e.g. '[2,1,1]'")
            args.optimized_mbs_list = sizes
            args.micro_batch_sizes = sizes
            args.micro_batch_size = max(sizes)       # what buffers and memory estimates are sized for
        args.pp_schedule = None
        if args.pp_schedule_list:
            import ast
            import json
            v = args.pp_schedule_list
            if isinstance(v, str):
                try:
                    v = json.loads(v)
                except ValueError:
                    v = ast.literal_eval(v)
            if not isinstance(v, dict) or not all(isinstance(x, (list, tuple)) for x in v.values()):
                raise AssertionError('--pp-schedule-list is a mapping like {"stage0": ["F1", "F2", "B1", "B2"], "stage1": [...]}')
            args.pp_schedule_list = args.pp_schedule = {k: list(x) for k, x in v.items()}
        if getattr(args, "expert_interval", 1) > 1:
            if getattr(args, "moe_model_type", "megatron_moe") != "deepspeed_moe":
                raise AssertionError("--expert-interval belongs to --moe-model-type deepspeed_moe; use --moe-layer-freq otherwise")
            n = args.expert_interval
            args.moe_layer_freq = str([1 if (i + 1) % n == 0 else 0 for i in range(args.num_layers)])

    def validate_args(self, args):
        if getattr(args, "ampipe_degree", 1) > 1:
            if not args.num_experts or getattr(args, "moe_model_type", "megatron_moe") != "deepspeed_moe":
                raise AssertionError("--ampipe-degree pipelines the DeepSpeed-style MoE behind the attention: it needs --num-experts "
                                     "and --moe-model-type deepspeed_moe")
            local = args.seq_length // max(1, getattr(args, "context_parallel_size", 1))
            if getattr(args, "sequence_parallel", False):
                local //= args.tensor_model_parallel_size
            if local % args.ampipe_degree != 0:
                raise AssertionError("the sequence length per rank must be divisible by --ampipe-degree")
            for other in ("use_nanopipe", "recompute_in_bubble", "recompute_in_advance", "adaptive_recompute_device_swap", "moe_fb_overlap"):
                if getattr(args, other, False):
                    raise AssertionError(f"--ampipe-degree is not combined with --{other.replace('_', '-')}")
        if getattr(args, "moe_adaptive_recompute_activation", False) and not args.num_experts:
            raise AssertionError("--moe-adaptive-recompute-activation needs a MoE model (--num-experts)")
        if getattr(args, "moe_adaptive_recompute_activation_scale", 2.0) <= 0:
            raise AssertionError("--moe-adaptive-recompute-activation-scale must be positive")
        if getattr(args, "micro_batch_sizes", None):
            if sum(args.micro_batch_sizes) * args.data_parallel_size != args.global_batch_size:
                raise AssertionError(f"--optimized-mbs-list {args.micro_batch_sizes} sums to {sum(args.micro_batch_sizes)} samples per "
                                     f"data-parallel rank; the global batch {args.global_batch_size} over {args.data_parallel_size} "
                                     "data-parallel ranks needs " + str(args.global_batch_size // args.data_parallel_size))
            for other in ("reset_attention_mask", "use_multiparameter_pipeline_model_parallel"):
                if getattr(args, other, False):
                    raise AssertionError(f"--optimized-mbs-list is not combined with --{other.replace('_', '-')}")
            if getattr(args, "schedules_method", None) in ("dualpipev", "dualpipe", "chimera"):
                raise AssertionError("--optimized-mbs-list works with the 1F1B and interleaved schedules")
        if getattr(args, "pp_schedule", None):
            if args.pipeline_model_parallel_size < 2 or getattr(args, "num_layers_per_virtual_pipeline_stage", None) \
                    or getattr(args, "schedules_method", None) in ("dualpipev", "dualpipe", "chimera"):
                raise AssertionError("--pp-schedule-list orders the steps of the non-interleaved pipeline: it needs pipeline "
                                     "parallelism without virtual stages and without --schedules-method")
            from ..parallel.pipeline.plan import plan_from_stage_lists
            n_mb = len(args.micro_batch_sizes) if getattr(args, "micro_batch_sizes", None) else \
                args.global_batch_size // (args.micro_batch_size * args.data_parallel_size)
            try:
                plan_from_stage_lists(args.pipeline_model_parallel_size, n_mb, args.pp_schedule)
            except (ValueError, RuntimeError) as e:
                raise AssertionError(f"--pp-schedule-list: {e}")
        if not (0.0 <= args.save_memory_ratio < 1.0):
            raise AssertionError("--save-memory-ratio is a fraction in [0, 1)")


class ProfileFeature(Feature):
    def __init__(self):
        super().__init__("profile", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--profile", action="store_true")
        add_arg(g, "--profile-step-start", type=int, default=10)
        add_arg(g, "--profile-step-end", type=int, default=12)
        add_arg(g, "--profile-level", type=str, default="level0", choices=["level0", "level1", "level2"])
        add_arg(g, "--profile-with-cpu", action="store_true")
        add_arg(g, "--profile-with-stack", action="store_true")
        add_arg(g, "--profile-with-memory", action="store_true")
        add_arg(g, "--profile-record-shapes", action="store_true")
        add_arg(g, "--profile-save-path", type=str, default="./profile_dir")
        add_arg(g, "--profile-ranks", nargs="+", type=int, default=[-1])


class TflopsCalculateFeature(Feature):
    def __init__(self):
        super().__init__("op-cal-tflops", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--op-cal-tflops", action="store_true", help="count FLOPs per step and log MFU / HFU")


class DeterministicFeature(Feature):
    def __init__(self):
        super().__init__("npu-deterministic", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--npu-deterministic", "--deterministic", dest="npu_deterministic", action="store_true")
        add_arg(g, "--npu-datadump", "--tensor-dump", dest="npu_datadump", action="store_true")
        add_arg(g, "--jit-compile", action="store_true")

    def configure(self, manager, args):
        if getattr(args, "npu_deterministic", False):
            from ..utils.determinism import enable_determinism
            enable_determinism(getattr(args, "seed", 1234))


class TokenizerFeature(Feature):
    def __init__(self):
        super().__init__("tokenizer", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--tokenizer-name-or-path", type=str, default=None)
        add_arg(g, "--tokenizer-not-use-fast", action="store_false", dest="tokenizer_use_fast")


# ======================================================================================
# tensor parallel
# ======================================================================================
class FusedTPCommFeature(Feature):
    """Fused all-gather->GEMM and GEMM->reduce-scatter kernels (the reference's MC2,
    mindspeed/features_manager/tensor_parallel/mc2.py:15-32)."""

    def __init__(self):
        super().__init__("use-ascend-mc2", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--use-ascend-mc2", "--use-fused-tp-comm", dest="use_ascend_mc2", action="store_true")
        add_arg(g, "--tp-recompute-all-gather", action="store_true",
                help="re-gather the sequence-parallel input in backward instead of keeping the gathered copy from forward")

    def validate_args(self, args):
        self.incompatible_check(args, "use_ascend_coc")
        if args.use_ascend_mc2:
            if not getattr(args, "sequence_parallel", False) or getattr(args, "tensor_model_parallel_size", 1) <= 1:
                raise AssertionError("fused TP communication needs --sequence-parallel and tensor parallel size > 1")

    def configure(self, manager, args):
        manager.set_slot("tp_comm_ops", "fused", owner=self.feature_name)
        from ..parallel.layers import set_keep_gathered_input
        set_keep_gathered_input(not args.tp_recompute_all_gather)


class ChunkedTPCommFeature(Feature):
    """Chunk-pipelined GEMM / collective (the reference's CoC, features_manager/tensor_parallel/locl_coc.py:14-27)."""

    def __init__(self):
        super().__init__("use-ascend-coc", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--use-ascend-coc", "--use-chunked-tp-comm", dest="use_ascend_coc", action="store_true")
        add_arg(g, "--coc-mode", type=int, default=-1, choices=[-1, 0, 1, 2])
        add_arg(g, "--coc-parallel-num", type=int, default=1, choices=[1, 2, 4, 8])
        add_arg(g, "--coc-fused-kernel", action="store_true")

    def validate_args(self, args):
        if args.use_ascend_coc and args.coc_fused_kernel and not getattr(args, "sequence_parallel", False):
            raise AssertionError("--coc-fused-kernel needs --sequence-parallel")

    def configure(self, manager, args):
        manager.set_slot("tp_comm_ops", "fused" if args.coc_fused_kernel else "chunked", owner=self.feature_name)


class TP2DFeature(Feature):
    def __init__(self):
        super().__init__("tp-2d", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--tp-2d", action="store_true")
        add_arg(g, "--tp-x", type=int, default=1)
        add_arg(g, "--tp-y", type=int, default=1)
        add_arg(g, "--enable-overlap-ag-with-matmul", action="store_true")
        add_arg(g, "--enable-overlap-matmul-with-rs", action="store_true")
        add_arg(g, "--enable-backward-overlap-ag-with-matmul", action="store_true")

    def validate_args(self, args):
        if not args.tp_2d:
            return
        if args.tp_x * args.tp_y != args.tensor_model_parallel_size:
            raise AssertionError("tp_x * tp_y must equal --tensor-model-parallel-size")
        for bad in ("sequence_parallel", "use_ascend_coc"):
            if getattr(args, bad, False):
                raise AssertionError(f"--tp-2d is incompatible with {bad}")
        if getattr(args, "num_experts", None):
            raise AssertionError("--tp-2d does not support MoE")
        if getattr(args, "context_parallel_size", 1) > 1 and args.context_parallel_algo not in ("megatron_cp_algo", "ulysses_cp_algo"):
            raise AssertionError("--tp-2d supports ring or Ulysses context parallelism only")


class UnalignedLinearFeature(Feature):
    def __init__(self):
        super().__init__("unaligned-linear", optimization_level=2)

    def register_args(self, parser):
        add_arg(parser.add_argument_group(title=self.feature_name), "--unaligned-linear", action="store_true")

    def validate_args(self, args):
        if args.unaligned_linear and getattr(args, "use_ascend_mc2", False):
            raise AssertionError("--unaligned-linear is incompatible with the fused TP communication kernels")


# ======================================================================================
# context parallel / attention
# ======================================================================================
class ContextParallelFeature(Feature):
    def __init__(self):
        super().__init__("context-parallel-size", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--context-parallel-algo", type=str, default="megatron_cp_algo",
                choices=["megatron_cp_algo", "ulysses_cp_algo", "hybrid_cp_algo", "hybrid_adaptive_cp_algo",
                         "adaptive_cp_algo", "kvallgather_cp_algo", "hamilton_cp_algo"])
        add_arg(g, "--hamilton-path-num", type=int, default=0,
                help="hamilton_cp_algo: number of edge-disjoint cycles the KV block is split over (0: as many as the "
                     "context-parallel size allows)")
        add_arg(g, "--cp-window-size", type=int, default=1)
        add_arg(g, "--attention-mask-type", type=str, default="causal", choices=["causal", "general"])
        add_arg(g, "--use-cp-send-recv-overlap", action="store_true")
        add_arg(g, "--megatron-cp-in-bnsd", action="store_true")
        add_arg(g, "--ulysses-degree-in-cp", type=int, default=None)
        add_arg(g, "--context-parallel-kv-cache-policy", type=str, default=None, choices=[None, "full", "half"])
        add_arg(g, "--context-parallel-cache-interval", type=int, default=0)
        add_arg(g, "--use-ulysses-allgather-kv", action="store_true")
        add_arg(g, "--attention-mask-on-cpu", action="store_true")
        add_arg(g, "--adaptive-cp-without-coarse", action="store_true")
        add_arg(g, "--adaptive-cp-dynamic-attn-mask", action="store_true")
        add_arg(g, "--adaptive-cp-only-reschedule", action="store_true")
        add_arg(g, "--adaptive-cp-manually-set-mask-list", action="store_true")

    def is_need_apply(self, args):
        return getattr(args, "context_parallel_size", 1) > 1 and self.optimization_level <= getattr(args, "optimization_level", 2) \
            or getattr(args, "context_parallel_size", 1) > 1

    def validate_args(self, args):
        cp = args.context_parallel_size
        if cp <= 1:
            return
        algo = args.context_parallel_algo
        seq = args.seq_length
        if algo == "megatron_cp_algo":
            if seq % (2 * cp) != 0:
                raise AssertionError("ring context parallel needs seq_length divisible by 2 * cp")
            w = args.cp_window_size
            if not (1 <= w < cp) and cp > 1 and w != 1:
                raise AssertionError("cp_window_size must satisfy 1 <= window < cp")
            if cp % w != 0:
                raise AssertionError("cp must be divisible by cp_window_size")
        if algo == "ulysses_cp_algo":
            heads = args.num_attention_heads
            if heads % (cp * args.tensor_model_parallel_size) != 0:
                raise AssertionError("Ulysses needs num_attention_heads divisible by cp * tp")
            if seq % cp != 0:
                raise AssertionError("Ulysses needs seq_length divisible by cp")
        if algo in ("hybrid_cp_algo", "hybrid_adaptive_cp_algo"):
            u = args.ulysses_degree_in_cp
            if u is None or cp % u != 0 or not (1 < u < cp):
                raise AssertionError("hybrid context parallel needs 1 < ulysses_degree_in_cp < cp dividing cp")
            ring = cp // u
            if seq % (2 * ring * u) != 0:
                raise AssertionError("hybrid context parallel needs seq_length divisible by 2 * cp")
        if algo == "kvallgather_cp_algo" and args.attention_mask_type != "causal":
            raise AssertionError("KV-allgather context parallel supports causal attention only")
        if algo == "hamilton_cp_algo":
            if args.attention_mask_type == "causal":
                raise AssertionError("Hamilton context parallel supports full attention only (--attention-mask-type general)")
            import math
            paths = sum(1 for s_ in range(1, cp) if math.gcd(s_, cp) == 1)
            if not (0 <= args.hamilton_path_num <= paths):
                raise AssertionError(f"--hamilton-path-num must be within 0..{paths} for context parallel size {cp}")
            if seq % cp != 0:
                raise AssertionError("Hamilton context parallel needs seq_length divisible by cp")


class FlashAttentionFeature(Feature):
    def __init__(self):
        super().__init__("use-flash-attn", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--attention-backend", type=str, default="auto", choices=["auto", "library", "sm100"],
                help="sm100: hand-written tcgen05 flash attention; library: cuDNN/flash via torch; auto: the faster of the two")
        add_arg(g, "--pre-tockens", type=int, default=65536)
        add_arg(g, "--next-tockens", type=int, default=0)
        add_arg(g, "--sparse-mode", type=int, default=0, choices=[0, 1, 2, 3, 4])
        add_arg(g, "--use-fusion-attn-v2", action="store_true")
        add_arg(g, "--square-alibi-mask", action="store_true")
        add_arg(g, "--fill-neg-inf", action="store_true")
        add_arg(g, "--alibi-fusion-attn-type", type=int, default=None, choices=[None, 0, 2, 3])
        add_arg(g, "--alibi-diagonal-opposite", action="store_true")
        add_arg(g, "--reset-attention-mask", action="store_true")
        add_arg(g, "--fix-sub-seq-length", type=int, default=-1)


class AlibiFeature(Feature):
    """ALiBi position bias (reference: mindspeed/features_manager/transformer/flash_attention/alibi_feature.py:9-90)."""

    def __init__(self):
        super().__init__("position-embedding-type", optimization_level=0)

    def is_need_apply(self, args) -> bool:
        return getattr(args, "position_embedding_type", None) == "alibi" or args.alibi_fusion_attn_type is not None \
            or args.alibi_diagonal_opposite

    def validate_args(self, args):
        if args.position_embedding_type != "alibi":
            raise AssertionError("--alibi-fusion-attn-type / --alibi-diagonal-opposite need --position-embedding-type alibi")
        if args.alibi_diagonal_opposite and args.alibi_fusion_attn_type == 3:
            raise AssertionError("--alibi-diagonal-opposite applies to the linear bias (--alibi-fusion-attn-type 0 or 2)")
        if args.context_parallel_size > 1:
            raise AssertionError("--position-embedding-type alibi is not combined with context parallelism")
        if getattr(args, "reset_attention_mask", False):
            raise AssertionError("--position-embedding-type alibi is not combined with --reset-attention-mask")


class SparseAttentionFeature(Feature):
    """DeepSeek sparse attention (reference: mindspeed/features_manager/transformer/experimental_attention_variant/dsa.py:5-50)."""

    def __init__(self):
        super().__init__("experimental-attention-variant", optimization_level=0)

    def is_need_apply(self, args) -> bool:
        return bool(args.experimental_attention_variant or args.use_dsa_absorb or args.use_fused_lightning_indexer
                    or args.use_fused_sparse_flash_attention or args.use_fused_lightning_indexer_kl_loss)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--experimental-attention-variant", type=str, default=None, choices=[None, "dsa"])
        add_arg(g, "--use-dsa-absorb", action="store_true")
        add_arg(g, "--use-fused-lightning-indexer", action="store_true")
        add_arg(g, "--use-fused-sparse-flash-attention", action="store_true")
        add_arg(g, "--use-fused-lightning-indexer-kl-loss", action="store_true")
        add_arg(g, "--dsa-indexer-n-heads", type=int, default=64)
        add_arg(g, "--dsa-indexer-head-dim", type=int, default=128)
        add_arg(g, "--dsa-indexer-topk", type=int, default=2048)
        add_arg(g, "--dsa-indexer-loss-coeff", type=float, default=1.0)

    def validate_args(self, args):
        fused = (args.use_fused_lightning_indexer, args.use_fused_sparse_flash_attention, args.use_fused_lightning_indexer_kl_loss)
        if args.experimental_attention_variant != "dsa":
            if args.use_dsa_absorb or any(fused):
                raise AssertionError("--use-dsa-absorb / --use-fused-lightning-indexer* / --use-fused-sparse-flash-attention "
                                     "need --experimental-attention-variant dsa")
            return
        if not getattr(args, "multi_head_latent_attention", False):
            raise AssertionError("--experimental-attention-variant dsa is built on --multi-head-latent-attention")
        if not args.qk_layernorm:
            raise AssertionError("--experimental-attention-variant dsa needs --qk-layernorm (the latent query / key norms)")
        if any(fused) and not (all(fused) and args.use_dsa_absorb):
            raise AssertionError("the fused sparse-attention operators come as a set: give --use-dsa-absorb, "
                                 "--use-fused-lightning-indexer, --use-fused-sparse-flash-attention and "
                                 "--use-fused-lightning-indexer-kl-loss together")
        if args.context_parallel_size > 1:
            raise AssertionError("--experimental-attention-variant dsa is not combined with context parallelism")


class MLAFeature(Feature):
    def __init__(self):
        super().__init__("multi-head-latent-attention", optimization_level=2)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--multi-head-latent-attention", "--multi-latent-attention", dest="multi_head_latent_attention",
                action="store_true")
        add_arg(g, "--q-lora-rank", type=int, default=None)
        add_arg(g, "--kv-lora-rank", type=int, default=512)
        add_arg(g, "--v-head-dim", type=int, default=128)
        add_arg(g, "--qk-rope-head-dim", "--qk-pos-emb-head-dim", dest="qk_rope_head_dim", type=int, default=64)
        add_arg(g, "--qk-nope-head-dim", "--qk-head-dim", dest="qk_nope_head_dim", type=int, default=128)
        add_arg(g, "--recompute-mla-up-proj", action="store_true", help="rebuild the q / kv up-projection outputs in backward")
        add_arg(g, "--mla-swap-core-attn-out", action="store_true", help="tensors the MLA core attention saves wait in host memory")
        add_arg(g, "--mla-mm-split", action="store_true")
        add_arg(g, "--mla-up-proj-tp-overlap", action="store_true")
        add_arg(g, "--mtp-mem-efficient-logits", action="store_true")
        add_arg(g, "--rope-scaling-type", type=str, default=None, choices=[None, "yarn"])
        add_arg(g, "--rope-scaling-factor", "--rotary-scaling-factor", dest="rope_scaling_factor", type=float, default=1.0)
        add_arg(g, "--rope-scaling-original-max-position-embeddings", type=int, default=4096)
        add_arg(g, "--rope-scaling-beta-fast", "--beta-fast", dest="rope_scaling_beta_fast", type=int, default=32)
        add_arg(g, "--rope-scaling-beta-slow", "--beta-slow", dest="rope_scaling_beta_slow", type=int, default=1)
        add_arg(g, "--rope-scaling-mscale", type=float, default=1.0)
        add_arg(g, "--rope-scaling-mscale-all-dim", type=float, default=0.0)


# ======================================================================================
# pipeline parallel
# ======================================================================================
class DualpipeVFeature(Feature):
    def __init__(self):
        super().__init__("schedules-method", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--schedules-method", type=str, default=None, choices=[None, "dualpipev", "dualpipe", "chimera"])
        add_arg(g, "--dualpipev-dw-detach", action="store_true")

    def validate_args(self, args):
        if args.schedules_method in ("dualpipev", "dualpipe"):
            pp = args.pipeline_model_parallel_size
            if pp < 2:
                raise AssertionError("DualPipe schedules need pipeline parallel size >= 2")
            if args.num_layers % (2 * pp) != 0:
                raise AssertionError("number of layers must be divisible by 2 * pipeline parallel size")
            nmb = args.global_batch_size // (args.micro_batch_size * max(1, args.data_parallel_size))
            if nmb < 2 * pp:
                raise AssertionError("DualPipe schedules need at least 2 * pp micro-batches")
            for bad in ("num_layers_per_virtual_pipeline_stage", "swap_attention", "tp_2d"):
                if getattr(args, bad, None):
                    raise AssertionError(f"dualpipe schedules are incompatible with {bad}")
            if getattr(args, "context_parallel_size", 1) > 1:
                raise AssertionError("dualpipe schedules are incompatible with context parallelism")

    def configure(self, manager, args):
        manager.set_slot("schedule", args.schedules_method, owner=self.feature_name)


class PipelineMiscFeature(Feature):
    def __init__(self):
        super().__init__("pipeline-misc", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--use-nanopipe", action="store_true",
                help="interleaved schedule: the first weight-gradient GEMMs of each rank run behind its last backward")
        add_arg(g, "--use-nanopipe-swap", action="store_true",
                help="--use-nanopipe: what the deferred weight gradients need waits in pinned host memory")
        add_arg(g, "--recompute-in-bubble", action="store_true")
        add_arg(g, "--recompute-in-advance", action="store_true")
        add_arg(g, "--noop-layers", type=str, default=None)
        add_arg(g, "--optimize-send-recv-comm", action="store_true")
        add_arg(g, "--use-multiparameter-pipeline-model-parallel", action="store_true")
        add_arg(g, "--pipeline-model-parallel-layout", type=str, default=None)
        add_arg(g, "--pipeline-num-transformer-layers", type=str, default=None)
        add_arg(g, "--automated-pipeline", action="store_true")
        add_arg(g, "--automated-pipeline-perf", action="store_true")
        add_arg(g, "--recompute-module-list", type=str, default=None,
                help="per pipeline rank: how many modules recompute, e.g. '[4,2,0,0]' (the policy an automated-pipeline run prints)")
        add_arg(g, "--recompute-type", type=int, default=2, choices=[0, 1, 2],
                help="what --recompute-module-list counts: 0 the MLP block, 1 the attention block, 2 whole transformer layers")
        add_arg(g, "--num-layer-list", type=str, default=None,
                help="transformer layers per pipeline rank, e.g. '[8,9,9,6]' (the layer policy an automated-pipeline run prints)")

    def validate_args(self, args):
        if args.use_multiparameter_pipeline_model_parallel and not getattr(args, "pipeline_tensor_shapes", None):
            # a model whose stages hand over several tensors sets args.pipeline_tensor_shapes itself; the default is the
            # one hidden-state tensor (reference: mindspeed/features_manager/pipeline_parallel/multi_parameter.py:38-52)
            import torch
            s_ = args.seq_length // max(1, getattr(args, "context_parallel_size", 1))
            if getattr(args, "sequence_parallel", False):
                s_ //= args.tensor_model_parallel_size
            dt = torch.bfloat16 if getattr(args, "bf16", False) else torch.float16 if getattr(args, "fp16", False) else torch.float32
            args.pipeline_tensor_shapes = [{"shape": (s_, args.micro_batch_size, args.hidden_size), "dtype": dt}]
        if args.use_nanopipe_swap and not args.use_nanopipe:
            raise AssertionError("--use-nanopipe-swap needs --use-nanopipe")
        if args.use_nanopipe:
            if getattr(args, "pipeline_model_parallel_size", 1) < 2 or not getattr(args, "num_layers_per_virtual_pipeline_stage", None):
                raise AssertionError("--use-nanopipe splits the backward of the interleaved schedule: it needs pipeline parallelism "
                                     "with --num-layers-per-virtual-pipeline-stage")
            for other in ("moe_fb_overlap", "tp_2d", "recompute_in_bubble", "recompute_in_advance"):
                if getattr(args, other, False):
                    raise AssertionError(f"--use-nanopipe is not combined with --{other.replace('_', '-')}")
            if getattr(args, "schedules_method", None) not in (None, "", "1f1b", "interleaved"):
                raise AssertionError("--use-nanopipe belongs to the interleaved schedule, not to --schedules-method "
                                     f"{args.schedules_method}")
        if args.recompute_in_bubble and args.recompute_in_advance:
            raise AssertionError("--recompute-in-bubble and --recompute-in-advance are exclusive")
        if (args.recompute_in_bubble or args.recompute_in_advance):
            if getattr(args, "pipeline_model_parallel_size", 1) < 2:
                raise AssertionError("recompute scheduling (--recompute-in-bubble / --recompute-in-advance) needs pipeline parallelism")
            if getattr(args, "schedules_method", None):
                raise AssertionError("recompute scheduling applies to the 1F1B and interleaved schedules only")
            if getattr(args, "recompute_granularity", None):
                # launch scripts give the schedule flag on top of --recompute-granularity full: the scheduler then places the
                # recompute of every layer it covers, so the in-backward recompute is switched off
                from ..utils.logging import print_rank_0
                print_rank_0("note: scheduler-placed recompute (--recompute-in-bubble / --recompute-in-advance) takes the place of "
                             "--recompute-granularity / --recompute-method / --recompute-num-layers")
                args.recompute_granularity, args.recompute_method, args.recompute_num_layers = None, None, None
        if isinstance(args.noop_layers, str):
            args.noop_layers = sorted({int(x) for x in args.noop_layers.split(",") if x != ""})
        if isinstance(args.pipeline_num_transformer_layers, str):
            import ast
            args.pipeline_num_transformer_layers = ast.literal_eval(args.pipeline_num_transformer_layers)
        for name in ("recompute_module_list", "num_layer_list"):
            v = getattr(args, name, None)
            if isinstance(v, str):
                import ast
                v = ast.literal_eval(v) if v.strip().startswith("[") else [int(x) for x in v.split(",") if x.strip() != ""]
                setattr(args, name, [int(x) for x in v])
        pp_ = getattr(args, "pipeline_model_parallel_size", 1)
        if args.num_layer_list:
            # a stored layer policy: same effect as --pipeline-num-transformer-layers
            if len(args.num_layer_list) != pp_ or sum(args.num_layer_list) != args.num_layers:
                raise AssertionError("--num-layer-list needs one entry per pipeline rank, summing to --num-layers")
            if not args.pipeline_num_transformer_layers:
                args.pipeline_num_transformer_layers = list(args.num_layer_list)
        if args.recompute_module_list:
            if len(args.recompute_module_list) != pp_:
                raise AssertionError("--recompute-module-list needs one entry per pipeline rank")
            if args.recompute_type == 2:
                if getattr(args, "recompute_granularity", None) not in (None, "full"):
                    raise AssertionError("--recompute-module-list with --recompute-type 2 is full-layer recompute")
                args.recompute_granularity, args.recompute_method = "full", "block"
                args.enable_recompute_layers_per_pp_rank = True
                args.recompute_num_layers = list(args.recompute_module_list)
            elif getattr(args, "recompute_granularity", None) == "full":
                raise AssertionError("--recompute-type 0 / 1 recompute one block of a layer; do not combine with full recompute")
        if args.automated_pipeline or args.automated_pipeline_perf:
            # layers per stage (and layers to recompute per stage) from the model shape, so that the stage that also holds
            # the output layer gets fewer transformer layers (reference: mindspeed/core/memory/auto_pipeline/*,
            # mindspeed/core/performance/auto_pipeline_perf/*); --automated-pipeline-perf also picks the micro-batch size
            pp = getattr(args, "pipeline_model_parallel_size", 1)
            if pp < 2:
                raise AssertionError("--automated-pipeline needs pipeline parallelism")
            if getattr(args, "num_layers_per_virtual_pipeline_stage", None) or getattr(args, "schedules_method", None) or \
                    args.pipeline_num_transformer_layers or getattr(args, "pipeline_model_parallel_layout", None):
                raise AssertionError("--automated-pipeline chooses the 1F1B layer split itself: no virtual stages, V / "
                                     "bidirectional schedules or hand-written layer lists")
            from ..memory.auto_pipeline import plan_from_args
            mbs, plan = plan_from_args(args, search_micro_batch_size=bool(args.automated_pipeline_perf))
            if not plan.feasible:
                raise AssertionError("--automated-pipeline: no layer split fits the memory budget")
            args.micro_batch_size = mbs
            args.pipeline_num_transformer_layers = list(plan.layers_per_stage)
            if any(plan.recompute_per_stage) and not getattr(args, "recompute_granularity", None):
                args.recompute_granularity, args.recompute_method = "full", "block"
                args.enable_recompute_layers_per_pp_rank = True
                args.recompute_num_layers = list(plan.recompute_per_stage)
            args.automated_pipeline_plan = plan

    def configure(self, manager, args):
        if args.recompute_in_bubble:
            manager.set_slot("schedule", "ripipe_bubble", owner=self.feature_name, force=True)
        elif args.recompute_in_advance:
            manager.set_slot("schedule", "ripipe_advance", owner=self.feature_name, force=True)


# ======================================================================================
# MoE
# ======================================================================================
class MoEFeature(Feature):
    def __init__(self):
        super().__init__("moe", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--moe-tp-extend-ep", action="store_true")
        add_arg(g, "--expert-interval", type=int, default=1,
                help="--moe-model-type deepspeed_moe: every expert-interval-th layer is a MoE layer")
        add_arg(g, "--enable-token-rearrange-opt", action="store_true")
        add_arg(g, "--use-rts", action="store_true", default=False,
                help="deepspeed_moe top-1 gate: over-capacity experts keep a random selection of their tokens")
        add_arg(g, "--no-use-rts", action="store_false", dest="use_rts")
        add_arg(g, "--moe-adaptive-recompute-activation", action="store_true",
                help="recompute a MoE layer in backward only on steps where its busiest expert is over scale x the balanced load")
        add_arg(g, "--moe-adaptive-recompute-activation-scale", type=float, default=2.0)
        add_arg(g, "--ampipe-tp-sp-comm-overlap", action="store_true")
        add_arg(g, "--moe-permutation-async-comm", action="store_true")
        add_arg(g, "--moe-alltoall-overlap-comm", action="store_true")
        add_arg(g, "--moe-allgather-overlap-comm", action="store_true")
        add_arg(g, "--moe-alltoall-mc2", "--moe-alltoall-fused", dest="moe_alltoall_mc2", action="store_true")
        add_arg(g, "--moe-fb-overlap", action="store_true")
        add_arg(g, "--moe-unperm2-mem-optim-swap", action="store_true")
        add_arg(g, "--moe-zero-memory", type=str, default="disable", choices=["disable", "level0", "level1"])
        add_arg(g, "--moe-zero-memory-num-layers", type=int, default=None)
        add_arg(g, "--n-shared-experts", type=int, default=None)
        add_arg(g, "--fix-router", action="store_true")
        add_arg(g, "--balanced-moe-experts", action="store_true")
        add_arg(g, "--balanced-moe-hot-expert-num", type=int, default=3)
        add_arg(g, "--trans-hot-expert-group-num", type=int, default=3)
        add_arg(g, "--enable-expert-placement", action="store_true")
        add_arg(g, "--expert-placement-freq", type=int, default=50)
        add_arg(g, "--enable-fine-grained-expert-placement", action="store_true")
        add_arg(g, "--fine-grained-expert-placement-thre", type=float, default=0.08)
        add_arg(g, "--print-expert-load", action="store_true")
        add_arg(g, "--moe-bmm-mc2", action="store_true")
        # legacy deepspeed-style MoE
        add_arg(g, "--moe-model-type", type=str, default="megatron_moe", choices=["deepspeed_moe", "megatron_moe"])
        add_arg(g, "--moe-train-capacity-factor", type=float, default=1.0)
        add_arg(g, "--noisy-gate-policy", type=str, default=None)
        add_arg(g, "--moe-no-drop", action="store_true")
        add_arg(g, "--moe-dynamic-padding", action="store_true")
        add_arg(g, "--moe-use-sinkhorn", action="store_true")
        add_arg(g, "--use-pipe-experts", action="store_true")
        add_arg(g, "--pipe-experts-multi-data", type=int, default=1)
        add_arg(g, "--pipe-experts-multi-stream", action="store_true")
        add_arg(g, "--ampipe-degree", type=int, default=1)

    def validate_args(self, args):
        ne = getattr(args, "num_experts", None)
        if args.moe_alltoall_overlap_comm or args.moe_alltoall_mc2:
            if getattr(args, "expert_model_parallel_size", 1) <= 1:
                raise AssertionError("the overlapped / fused alltoall dispatcher needs expert parallel size > 1")
            if not getattr(args, "moe_grouped_gemm", False):
                raise AssertionError("the overlapped / fused alltoall dispatcher needs --moe-grouped-gemm")
            if getattr(args, "moe_token_dispatcher_type", "alltoall") not in ("alltoall", "alltoall_seq"):
                raise AssertionError("alltoall overlap needs --moe-token-dispatcher-type alltoall")
        if args.moe_bmm_mc2:
            # the reference's fused all-to-all + batched-matmul op pair; here the same role is played by the peer-memory
            # dispatch / combine kernels around the one-launch grouped GEMM
            if getattr(args, "expert_model_parallel_size", 1) <= 1 or not getattr(args, "moe_grouped_gemm", False):
                raise AssertionError("--moe-bmm-mc2 needs expert parallel size > 1 and --moe-grouped-gemm")
            args.moe_alltoall_mc2 = True
        legacy = getattr(args, "moe_model_type", "megatron_moe") == "deepspeed_moe"
        if (args.use_pipe_experts or args.pipe_experts_multi_data > 1 or args.pipe_experts_multi_stream) and not legacy:
            raise AssertionError("pipelined experts (--use-pipe-experts, --pipe-experts-*) belong to --moe-model-type deepspeed_moe")
        if legacy:
            if not ne:
                raise AssertionError("--moe-model-type deepspeed_moe needs --num-experts")
            if getattr(args, "moe_router_topk", 2) not in (1, 2):
                raise AssertionError("the DeepSpeed-style gate supports --moe-router-topk 1 or 2")
            if args.moe_alltoall_mc2 or args.moe_alltoall_overlap_comm or args.moe_fb_overlap or args.balanced_moe_experts:
                raise AssertionError("--moe-model-type deepspeed_moe has its own dispatch (einsum + all-to-all); the core "
                                     "dispatcher options do not apply to it")
        if args.enable_fine_grained_expert_placement and not args.enable_expert_placement:
            raise AssertionError("--enable-fine-grained-expert-placement refines --enable-expert-placement: set both")
        if args.balanced_moe_experts:
            if getattr(args, "expert_model_parallel_size", 1) <= 1 or not getattr(args, "moe_grouped_gemm", False):
                raise AssertionError("--balanced-moe-experts needs expert parallel size > 1 and --moe-grouped-gemm")
            if args.moe_alltoall_mc2:
                raise AssertionError("--balanced-moe-experts leaves tokens with fewer than top-k remote experts; the fused "
                                     "dispatcher (--moe-alltoall-mc2) needs exactly top-k per token")
            if getattr(args, "use_fused_dist_opt", False) or getattr(args, "ddp_average_in_collective", False):
                raise AssertionError("--balanced-moe-experts adds the replicas' gradients after the data-parallel reduction; "
                                     "it is not combined with --use-fused-dist-opt or --ddp-average-in-collective")
            if ne and not (0 < args.balanced_moe_hot_expert_num <= ne):
                raise AssertionError("--balanced-moe-hot-expert-num must be within 1..num_experts")
        if args.moe_allgather_overlap_comm and getattr(args, "moe_token_dispatcher_type", "alltoall") != "allgather":
            raise AssertionError("--moe-allgather-overlap-comm needs --moe-token-dispatcher-type allgather")
        if args.moe_fb_overlap:
            if getattr(args, "moe_token_dispatcher_type", "") != "alltoall" or not getattr(args, "moe_grouped_gemm", False):
                raise AssertionError("--moe-fb-overlap needs the alltoall dispatcher and grouped GEMM")
            if (getattr(args, "expert_tensor_parallel_size", None) or 1) != 1:
                raise AssertionError("--moe-fb-overlap needs expert tensor parallel size 1")
            if getattr(args, "moe_pad_expert_input_to_capacity", False):
                raise AssertionError("--moe-fb-overlap does not support drop-and-pad")
            if getattr(args, "pipeline_model_parallel_size", 1) > 1 and (
                    getattr(args, "recompute_in_bubble", False) or getattr(args, "recompute_in_advance", False) or
                    getattr(args, "schedules_method", None) in ("dualpipe", "chimera") or
                    getattr(args, "use_multiparameter_pipeline_model_parallel", False)):
                raise AssertionError("--moe-fb-overlap with pipeline parallelism runs on the 1F1B, interleaved and DualPipeV "
                                     "schedules, without scheduler-placed recompute or list-valued stage interfaces")
            if getattr(args, "recompute_granularity", None) == "full":
                raise AssertionError("--moe-fb-overlap keeps the staged layer graphs: no full recompute")
        if args.moe_alltoall_mc2 and getattr(args, "use_ascend_mc2", False) and ne:
            pass
        if args.moe_tp_extend_ep and ne and ne % (getattr(args, "tensor_model_parallel_size", 1) *
                                                   getattr(args, "expert_model_parallel_size", 1)) != 0:
            raise AssertionError("--moe-tp-extend-ep needs num_experts divisible by tp * ep")

    def configure(self, manager, args):
        if args.moe_alltoall_mc2:
            manager.set_slot("moe_dispatcher", "fused", owner=self.feature_name)
        elif args.moe_alltoall_overlap_comm:
            manager.set_slot("moe_dispatcher", "overlap", owner=self.feature_name)


# ======================================================================================
# memory
# ======================================================================================
class MemoryFeature(Feature):
    def __init__(self):
        super().__init__("memory", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--recompute-activation-function", action="store_true")
        add_arg(g, "--recompute-activation-function-num-layers", type=int, default=None)
        add_arg(g, "--recompute-norm", action="store_true")
        add_arg(g, "--recompute-norm-num-layers", type=int, default=None)
        add_arg(g, "--enable-recompute-layers-per-pp-rank", action="store_true")
        add_arg(g, "--swap-attention", action="store_true")
        add_arg(g, "--swap-modules", type=str, default="input_norm,self_attention,post_attention_norm")
        add_arg(g, "--swap-layer-input", action="store_true")
        add_arg(g, "--smart-swap", action="store_true")
        add_arg(g, "--reuse-fp32-param", action="store_true")
        add_arg(g, "--compress-dense", type=str, default="disable", choices=["disable", "level0", "level1"])
        add_arg(g, "--compress-activation", type=str, default="",
                help='layers whose saved activations are stored compressed: "0" = all, or e.g. "1,3-5" (1-based)')
        add_arg(g, "--compress-optimizer", action="store_true")
        add_arg(g, "--adaptive-recompute-device-size", type=int, default=-1)
        add_arg(g, "--adaptive-recompute-profiling-step", type=int, default=10)
        add_arg(g, "--adaptive-recompute-device-swap", action="store_true")
        add_arg(g, "--adaptive-memory-optimization", action="store_true")

    def validate_args(self, args):
        if args.swap_attention and getattr(args, "schedules_method", None) in ("dualpipev", "dualpipe"):
            raise AssertionError("--swap-attention is incompatible with dualpipe schedules")
        if args.reuse_fp32_param and getattr(args, "optimizer_selection", "") == "fused_ema_adamw":
            raise AssertionError("--reuse-fp32-param is incompatible with fused_ema_adamw")
        if args.reuse_fp32_param and not getattr(args, "bf16", False):
            raise AssertionError("--reuse-fp32-param needs --bf16")
        if args.compress_activation not in ("", None):
            from ..memory.compress_activation import parse_layers
            args.compress_activation = parse_layers(args.compress_activation, args.num_layers)
            if getattr(args, "recompute_granularity", None) == "full":
                raise AssertionError("--compress-activation stores what a layer saves for backward; full recompute saves nothing")
        else:
            args.compress_activation = []
        if args.smart_swap and (args.swap_attention or args.adaptive_memory_optimization):
            raise AssertionError("--smart-swap excludes --swap-attention / --adaptive-memory-optimization")


# ======================================================================================
# optimizer
# ======================================================================================
class OptimizerFeature(Feature):
    def __init__(self):
        super().__init__("optimizer", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--swap-optimizer", action="store_true")
        add_arg(g, "--swap-optimizer-times", type=int, default=16)
        add_arg(g, "--virtual-optimizer", nargs="+", type=float, default=None)
        add_arg(g, "--quant-states", type=str, default=None, choices=[None, "fp8", "hif8", "mxfp8"])
        add_arg(g, "--quant-grads", action="store_true")
        add_arg(g, "--ema-decay", type=float, default=0.9999)
        add_arg(g, "--use-ema", action="store_true")
        for name, typ, default in (("--muon-momentum", float, 0.95), ("--muon-num-ns-steps", int, 5),
                                   ("--muon-extra-scale-factor", float, 1.0)):
            add_arg(g, name, type=typ, default=default)
        add_arg(g, "--muon-nesterov", action="store_true")
        add_arg(g, "--muon-scale-mode", type=str, default="spectral", choices=["spectral", "unit_rms_norm", "shape_scaling"])
        add_arg(g, "--muon-tp-mode", type=str, default="blockwise", choices=["blockwise", "duplicated", "distributed"])
        add_arg(g, "--muon-coefficient-type", type=str, default="quintic", choices=["simple", "quintic", "polar_express"])
        add_arg(g, "--muon-fp32-matmul-prec", type=str, default="medium", choices=["low", "medium", "high"])
        add_arg(g, "--muon-scalar-optimizer", type=str, default="adam")
        add_arg(g, "--muon-no-split-qkv", action="store_false", dest="muon_split_qkv")
        add_arg(g, "--apply-wd-to-qk-layernorm", action="store_true")

    def validate_args(self, args):
        if getattr(args, "compress_optimizer", False) and (args.swap_optimizer or args.quant_states or
                                                          getattr(args, "use_fused_dist_opt", False) or getattr(args, "virtual_optimizer", None)):
            raise AssertionError("--compress-optimizer keeps the moments encoded between steps; it is not combined with "
                                 "--swap-optimizer, --quant-states, --virtual-optimizer or --use-fused-dist-opt")
        if getattr(args, "quant_grads", False):
            if getattr(args, "gradient_accumulation_fusion", False):
                raise AssertionError("--quant-grads keeps 16-bit gradient buffers; the GEMM epilogue accumulates into fp32 "
                                     "buffers: add --no-gradient-accumulation-fusion")
            if args.swap_optimizer or getattr(args, "use_fused_dist_opt", False):
                raise AssertionError("--quant-grads is not combined with --swap-optimizer or --use-fused-dist-opt")
        if args.swap_optimizer and args.quant_states:
            raise AssertionError("--swap-optimizer is incompatible with the low-precision optimizer")
        if args.quant_states == "hif8":
            raise AssertionError("hif8 optimizer states are Ascend-specific; use fp8 or mxfp8")


# ======================================================================================
# distributed
# ======================================================================================
class DistributedFeature(Feature):
    def __init__(self):
        super().__init__("distributed", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--param-and-grad-buffer-pad", type=int, default=None)
        add_arg(g, "--reset-bucket-group-order", action="store_true")
        add_arg(g, "--layerzero", action="store_true")
        add_arg(g, "--layerzero-config", type=str, default=None)
        add_arg(g, "--fsdp2-config-path", type=str, default=None)
        add_arg(g, "--disable-gloo-group", action="store_true")
        add_arg(g, "--hccl-slice-size", "--nccl-slice-size", dest="hccl_slice_size", type=int, default=10 * 1024 * 1024)
        add_arg(g, "--hccl-group-buffer", "--nccl-group-buffer", dest="hccl_group_buffer", type=str, default=None)
        add_arg(g, "--hccl-group-buffer-adaptive", action="store_true")
        add_arg(g, "--hccl-ep-group-buffer-adaptive-factor", type=float, default=-1.0)
        add_arg(g, "--hccl-op-mode", type=str, default=None)
        add_arg(g, "--async-log-allreduce", action="store_true")
        add_arg(g, "--no-fused-ulysses-a2a", action="store_true",
                help="level 2 runs the Ulysses all-to-alls as peer-memory kernels with the layout transform fused in; this keeps NCCL")
        add_arg(g, "--use-fused-dist-opt", action="store_true",
                help="distributed-optimizer step as one peer-memory kernel (reduce-scatter + AdamW + all-gather); "
                     "needs --use-distributed-optimizer, a data-parallel group of 2..8 GPUs in one NVSwitch domain and level 2")
        add_arg(g, "--dist-train", action="store_true")
        add_arg(g, "--aiqos", action="store_true")
        add_arg(g, "--aiqos-mode", type=str, default="auto")
        add_arg(g, "--aiqos-schedule", type=str, default=None)
        add_arg(g, "--aiqos-enable-roce", action="store_true")

    def validate_args(self, args):
        if args.param_and_grad_buffer_pad is not None and args.param_and_grad_buffer_pad <= 0:
            raise AssertionError("--param-and-grad-buffer-pad must be positive")
        if args.layerzero and getattr(args, "use_distributed_optimizer", False):
            raise AssertionError("--layerzero replaces --use-distributed-optimizer")


class AutoSettingsFeature(Feature):
    def __init__(self):
        super().__init__("auto-settings", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--auto-settings", action="store_true")
        add_arg(g, "--auto-settings-work-dir", type=str, default="./auto_settings_dir")
        add_arg(g, "--auto-settings-ranks", type=int, default=8)
        add_arg(g, "--auto-settings-log-level", type=str, default="info", choices=["debug", "info", "warning"])
        add_arg(g, "--auto-settings-type", type=str, default="white", choices=["white", "black", "mixed"])
        add_arg(g, "--target-nnodes", type=int, default=1)
        add_arg(g, "--nnodes", type=int, default=1)
        add_arg(g, "--nproc-per-node", type=int, default=8)
        add_arg(g, "--node-rank", type=int, default=0)
        add_arg(g, "--master-addr", type=str, default="127.0.0.1")
        add_arg(g, "--master-port", type=int, default=12345)
        add_arg(g, "--prof-file", type=str, default=None)


class TTPFeature(Feature):
    def __init__(self):
        super().__init__("ttp-enabled", optimization_level=0)

    def register_args(self, parser):
        g = parser.add_argument_group(title=self.feature_name)
        add_arg(g, "--ttp-enabled", action="store_true")
        add_arg(g, "--ttp-server-ip", type=str, default="127.0.0.1")
        add_arg(g, "--ttp-server-port", type=int, default=29500)
        add_arg(g, "--ttp-dump-dir", type=str, default=None)
        add_arg(g, "--ttp-max-dump-ckpt-to-keep", type=int, default=1)
        add_arg(g, "--ttp-save-optimizer", action="store_true")
        add_arg(g, "--ttp-save-rng", action="store_true")
        add_arg(g, "--ttp-dump-timeout-seconds", type=int, default=60)
        add_arg(g, "--ttp-wait-dump-file-timeout", type=int, default=60)
        add_arg(g, "--ttp-heartbeat-interval-ms", type=int, default=1000)
        add_arg(g, "--ttp-heartbeat-timeout-ms", type=int, default=3000)
        add_arg(g, "--ttp-max-missed-count", type=int, default=3)

    def validate_args(self, args):
        if args.ttp_enabled and not args.ttp_dump_dir:
            raise AssertionError("--ttp-enabled needs --ttp-dump-dir")


def create_features_list():
    return [
        RequirementsBasicFeature(), MegatronBasicFeature(), TransformerEngineBasicFeature(), LegacySpellingsFeature(), QADFeature(), ProfileFeature(),
        TflopsCalculateFeature(), DeterministicFeature(), TokenizerFeature(),
        FusedTPCommFeature(), ChunkedTPCommFeature(), TP2DFeature(), UnalignedLinearFeature(),
        ContextParallelFeature(), FlashAttentionFeature(), AlibiFeature(), SparseAttentionFeature(), MLAFeature(),
        DualpipeVFeature(), PipelineMiscFeature(), MoEFeature(), MemoryFeature(), OptimizerFeature(),
        DistributedFeature(), AutoSettingsFeature(), TTPFeature(),
    ]
