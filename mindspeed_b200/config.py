"""Model / parallel configuration dataclasses.

``TransformerConfig`` follows the field names of Megatron-core 0.12's
``TransformerConfig`` / ``ModelParallelConfig`` so that model code written against
Megatron reads the same attributes.  Every command-line flag is also mirrored onto
the config object as a dynamic attribute (``config.<flag>``), the behaviour the
reference obtains by rewriting the dataclass at import time
(reference: mindspeed/core/megatron_basic/arguments_basic.py:88-137).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.nn.functional as F


@dataclass
class ModelParallelConfig:
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    context_parallel_size: int = 1
    hierarchical_context_parallel_sizes: Optional[List[int]] = None
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    moe_extended_tp: bool = False

    perform_initialization: bool = True
    use_cpu_initialization: bool = False
    fp16: bool = False
    bf16: bool = False
    params_dtype: torch.dtype = torch.float32
    timers: Optional[Callable] = None
    finalize_model_grads_func: Optional[Callable] = None
    # 2-D tensor parallelism: tensor_model_parallel_size = tp_x * tp_y
    tp_2d: bool = False
    tp_x: int = 1
    tp_y: int = 1
    grad_scale_func: Optional[Callable] = None
    no_sync_func: Optional[Callable] = None
    grad_sync_func: Optional[Callable] = None
    param_sync_func: Optional[Callable] = None
    deterministic_mode: bool = False
    enable_autocast: bool = False
    autocast_dtype: Optional[torch.dtype] = None
    num_microbatches_with_partial_activation_checkpoints: Optional[int] = None

    gradient_accumulation_fusion: bool = False
    async_tensor_model_parallel_allreduce: bool = False
    use_te_rng_tracker: bool = False
    tp_comm_overlap: bool = False
    tp_comm_bulk_wgrad: bool = True
    tp_comm_bulk_dgrad: bool = True
    tp_comm_overlap_ag: bool = True
    tp_comm_overlap_rs: bool = True
    cross_entropy_loss_fusion: bool = False

    pipeline_dtype: Optional[torch.dtype] = None
    variable_seq_lengths: bool = False
    overlap_p2p_comm: bool = False
    batch_p2p_comm: bool = True
    batch_p2p_sync: bool = True
    use_ring_exchange_p2p: bool = False
    deallocate_pipeline_outputs: bool = False
    defer_embedding_wgrad_compute: bool = False
    wgrad_deferral_limit: int = 0
    pipeline_model_parallel_split_rank: Optional[int] = None
    overlap_p2p_comm_warmup_flush: bool = False
    microbatch_group_size_per_vp_stage: Optional[int] = None

    cpu_offloading: bool = False
    cpu_offloading_num_layers: int = 0
    barrier_with_L1_time: bool = True


def _init_normal(sigma):
    def init_(t):
        return torch.nn.init.normal_(t, mean=0.0, std=sigma)

    return init_


def _scaled_init_normal(sigma, num_layers, multiplier=2.0):
    std = sigma / (multiplier * num_layers) ** 0.5

    def init_(t):
        return torch.nn.init.normal_(t, mean=0.0, std=std)

    return init_


@dataclass
class TransformerConfig(ModelParallelConfig):
    # ---- architecture ----
    num_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_query_groups: Optional[int] = None
    ffn_hidden_size: Optional[int] = None
    kv_channels: Optional[int] = None
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    fp32_residual_connection: bool = False
    apply_residual_connection_post_layernorm: bool = False
    layernorm_epsilon: float = 1e-5
    layernorm_zero_centered_gamma: bool = False
    add_bias_linear: bool = True
    add_qkv_bias: bool = False
    gated_linear_unit: bool = False
    activation_func: Callable = F.gelu
    activation_func_fp8_input_store: bool = False
    num_moe_experts: Optional[int] = None
    rotary_interleaved: bool = False
    window_size: Optional[Tuple[int, int]] = None            # (left, right) keys a query sees; -1 = unbounded
    pre_tockens: int = 65536                                 # the reference's spelling of the same bounds: keys before ...
    next_tockens: int = 0                                    # ... and after the query (sparse_mode 0 / 4)
    sparse_mode: int = 0                                     # 0 / 4: honour the bounds; 2 / 3: plain causal
    normalization: str = "LayerNorm"
    qk_layernorm: bool = False
    test_mode: bool = False
    calculate_per_token_loss: bool = False
    multi_latent_attention: bool = False
    position_embedding_type: str = "learned_absolute"        # "alibi": attention adds the per-head linear distance bias
    alibi_fusion_attn_type: Optional[int] = None             # None / 0 / 2: -slope * |i - j|; 3: -slope * sqrt|i - j|
    alibi_diagonal_opposite: bool = False                    # bias slope * (j - i): opposite signs on the two sides
    experimental_attention_variant: Optional[str] = None     # "dsa": lightning indexer + top-k sparse attention (MLA only)
    dsa_indexer_n_heads: int = 64
    dsa_indexer_head_dim: int = 128
    dsa_indexer_topk: int = 2048
    dsa_indexer_loss_coeff: float = 1.0
    use_dsa_absorb: bool = False
    kl_loss_reduction: str = "mean"
    softmax_scale: Optional[float] = None
    attention_softmax_in_fp32: bool = True
    apply_query_key_layer_scaling: bool = False
    masked_softmax_fusion: bool = True
    first_pipeline_num_layers: Optional[int] = None
    last_pipeline_num_layers: Optional[int] = None
    account_for_embedding_in_pipeline_split: bool = False
    account_for_loss_in_pipeline_split: bool = False

    # ---- init ----
    init_method: Optional[Callable] = None
    output_layer_init_method: Optional[Callable] = None
    init_method_std: float = 0.02

    # ---- fusion switches (level-1 single-GPU kernels) ----
    bias_activation_fusion: bool = False
    bias_dropout_fusion: bool = False
    apply_rope_fusion: bool = False
    use_fused_rmsnorm: bool = False
    use_fused_swiglu: bool = False
    use_fused_rotary_pos_emb: bool = False
    use_flash_attn: bool = False

    # ---- recompute ----
    recompute_granularity: Optional[str] = None
    recompute_method: Optional[str] = None
    recompute_num_layers: Optional[int] = None
    distribute_saved_activations: bool = False
    recompute_modules: Optional[List[str]] = None

    # ---- fp8 ----
    fp8: Optional[str] = None
    fp8_recipe: str = "delayed"
    fp8_margin: int = 0
    fp8_interval: int = 1
    fp8_amax_history_len: int = 1
    fp8_amax_compute_algo: str = "most_recent"
    fp8_wgrad: bool = True
    fp8_dot_product_attention: bool = False
    fp8_multi_head_attention: bool = False
    tp_only_amax_red: bool = False

    # ---- MoE ----
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_shared_expert_overlap: bool = False
    moe_layer_freq: Union[int, List[int]] = 1
    moe_ffn_hidden_size: Optional[int] = None
    moe_router_load_balancing_type: str = "aux_loss"
    moe_router_topk: int = 2
    moe_router_topk_limited_devices: Optional[int] = None
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_pre_softmax: bool = False
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_score_function: str = "softmax"
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3
    moe_router_dtype: Optional[str] = None
    moe_grouped_gemm: bool = False
    moe_use_legacy_grouped_gemm: bool = False
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: Optional[float] = None
    moe_input_jitter_eps: Optional[float] = None
    moe_token_dropping: bool = False
    moe_token_dispatcher_type: str = "allgather"
    moe_enable_deepep: bool = False
    moe_per_layer_logging: bool = False
    moe_expert_capacity_factor: Optional[float] = None
    moe_pad_expert_input_to_capacity: bool = False
    moe_token_drop_policy: str = "probs"
    moe_layer_recompute: bool = False
    moe_permute_fusion: bool = False
    first_k_dense_replace: int = 0

    # ---- MTP ----
    mtp_num_layers: Optional[int] = None
    mtp_loss_scaling_factor: Optional[float] = None

    # ---- context parallel ----
    cp_comm_type: Optional[Union[str, List[str]]] = None
    context_parallel_algo: str = "megatron_cp_algo"
    attention_mask_type: str = "causal"

    # ---- misc ----
    enable_cuda_graph: bool = False
    cuda_graph_retain_backward_graph: bool = False
    external_cuda_graph: bool = False
    clone_scatter_output_in_embedding: bool = True
    disable_parameter_transpose_cache: bool = False
    config_logger_dir: str = ""
    flash_decode: bool = False
    inference_rng_tracker: bool = False
    optimization_level: int = 2

    def __post_init__(self):
        if self.fp16 and self.bf16:
            raise ValueError("only one of fp16 / bf16 may be set")
        if self.num_attention_heads and self.num_attention_heads % max(1, self.tensor_model_parallel_size) != 0 \
                and not getattr(self, "unaligned_linear", False):
            raise ValueError("num_attention_heads must be divisible by tensor_model_parallel_size")
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.kv_channels is None and self.num_attention_heads:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        head_split = self.tp_x if self.tp_2d else self.tensor_model_parallel_size     # 2-D: heads split over tp-x only
        if self.num_query_groups and self.num_query_groups % max(1, head_split) != 0 \
                and not getattr(self, "unaligned_linear", False):
            raise ValueError("num_query_groups must be divisible by tensor_model_parallel_size (tp_x with --tp-2d)")
        if self.apply_query_key_layer_scaling:
            self.attention_softmax_in_fp32 = True
        if self.expert_model_parallel_size > 1 and self.num_moe_experts is None:
            raise ValueError("num_moe_experts must be set to use expert parallelism")
        if self.num_moe_experts is not None and self.num_moe_experts <= 0:
            raise ValueError("num_moe_experts must be positive")
        if self.moe_ffn_hidden_size is None:
            self.moe_ffn_hidden_size = self.ffn_hidden_size
        if self.moe_expert_capacity_factor is not None:
            if self.moe_token_dispatcher_type not in ("alltoall", "alltoall_seq"):
                raise ValueError("moe_expert_capacity_factor needs an alltoall dispatcher")
            if self.moe_expert_capacity_factor < 0:
                self.moe_expert_capacity_factor = None
        if self.moe_pad_expert_input_to_capacity and self.moe_expert_capacity_factor is None:
            raise ValueError("moe_pad_expert_input_to_capacity needs moe_expert_capacity_factor")
        if self.cpu_offloading and not (0 <= self.cpu_offloading_num_layers < self.num_layers):
            raise ValueError("cpu_offloading_num_layers out of range")
        if self.recompute_granularity is not None:
            if self.recompute_granularity not in ("full", "selective"):
                raise ValueError("recompute_granularity must be 'full' or 'selective'")
            if self.recompute_method is not None and self.recompute_method not in ("block", "uniform"):
                raise ValueError("recompute_method must be 'block' or 'uniform'")
            if self.recompute_granularity == "full" and self.recompute_method is None:
                raise ValueError("full recompute needs recompute_method")
            if self.recompute_granularity == "full" and self.recompute_num_layers is None:
                raise ValueError("full recompute needs recompute_num_layers")
        if self.virtual_pipeline_model_parallel_size is not None and self.num_layers:
            per = self.num_layers // self.pipeline_model_parallel_size
            if per % self.virtual_pipeline_model_parallel_size != 0 and not getattr(self, "pipeline_model_parallel_layout", None):
                raise ValueError("layers per pipeline stage must be divisible by the virtual pipeline size")
        if self.bias_activation_fusion and self.activation_func not in (F.gelu, F.silu):
            raise ValueError("bias_activation_fusion supports gelu and silu only")
        if self.init_method is None:
            self.init_method = _init_normal(self.init_method_std)
        if self.output_layer_init_method is None:
            self.output_layer_init_method = _scaled_init_normal(self.init_method_std, max(1, self.num_layers))
        if self.pipeline_dtype is None:
            self.pipeline_dtype = self.params_dtype
        if self.num_moe_experts is not None and self.moe_router_topk > self.num_moe_experts:
            raise ValueError("moe_router_topk exceeds num_moe_experts")

    # dynamic attributes: anything not declared above (every CLI flag) is kept as-is
    def update_from_args(self, args) -> "TransformerConfig":
        declared = {f.name for f in dataclasses.fields(self)}
        for k, v in vars(args).items():
            if k not in declared:
                object.__setattr__(self, k, v)
        return self


@dataclass
class MLATransformerConfig(TransformerConfig):
    """Multi-head latent attention (DeepSeek-V2/V3)."""
    multi_latent_attention: bool = True
    recompute_mla_up_proj: bool = False       # rebuild the q / kv up-projection outputs in backward
    mla_swap_core_attn_out: bool = False      # tensors the core attention saves wait in pinned host memory
    q_lora_rank: Optional[int] = 512
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    rope_type: str = "yarn"
    rotary_base: float = 10000
    rotary_percent: float = 1.0
    rotary_scaling_factor: float = 40
    max_position_embeddings: int = 4096
    original_max_position_embeddings: int = 4096
    beta_fast: float = 32
    beta_slow: float = 1
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    normalization: str = "RMSNorm"
