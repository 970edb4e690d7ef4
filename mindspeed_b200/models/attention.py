"""Self attention (MHA / GQA) and multi-head latent attention.

The QKV projection output keeps Megatron's packed layout ``[s, b, groups, (q_per_group + 2) * d]``
(checkpoint compatible).  Rotary embedding is applied in place on the q and k heads of that
buffer and the flash-attention kernel reads q / k / v as strided views of it, so no split copies
are made on the fused path.

Core attention dispatch with context parallelism mirrors the reference's
``CPDotProductAttentionImpl.forward`` (mindspeed/core/context_parallel/dot_product_attention.py:134-322).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops.rope import apply_rope, rope_packed_qkv_
from ..parallel import parallel_state as ps
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, divide, linear_classes
from ..parallel.random import get_cuda_rng_tracker
from .norms import build_norm


class _PackedRope(torch.autograd.Function):
    """In-place rotary on the q/k heads of packed QKV; backward rotates the gradient in place."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, groups, qpg, d, interleaved):
        ctx.save_for_backward(cos, sin)
        ctx.meta = (groups, qpg, d, interleaved)
        ctx.mark_dirty(qkv)
        rope_packed_qkv_(qkv, cos, sin, groups, qpg, d, interleaved, backward=False)
        return qkv

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        groups, qpg, d, interleaved = ctx.meta
        g = g.contiguous().clone() if not g.is_contiguous() else g.clone()
        rope_packed_qkv_(g, cos, sin, groups, qpg, d, interleaved, backward=True)
        return g, None, None, None, None, None, None


class CoreAttention(nn.Module):
    """softmax(QK^T / sqrt(d)) V with causal masking; context-parallel aware."""

    def __init__(self, config, layer_number=1, attn_mask_type="causal", softmax_scale=None, k_channels=None, v_channels=None):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        self.causal = attn_mask_type == "causal"
        d = k_channels or config.kv_channels
        self.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
        if config.apply_query_key_layer_scaling:
            self.softmax_scale /= layer_number
        self.dropout_p = config.attention_dropout
        self.alibi_slopes = None
        if getattr(config, "position_embedding_type", None) == "alibi":
            from .attention_masks import alibi_slopes
            tp, r = ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank()
            per = config.num_attention_heads // tp
            self.alibi_slopes = alibi_slopes(config.num_attention_heads)[r * per:(r + 1) * per]

    def _alibi(self, q, k, v, packed):
        if packed or ps.get_context_parallel_world_size() > 1:
            raise NotImplementedError("ALiBi attention is not combined with packed sequences or context parallelism")
        cfg = self.config
        self.alibi_slopes = self.alibi_slopes.to(q.device)
        return attn_ops.alibi_attention(q, k, v, self.alibi_slopes, causal=self.causal, softmax_scale=self.softmax_scale,
                                        mode=cfg.alibi_fusion_attn_type or 0, signed=bool(cfg.alibi_diagonal_opposite))

    def _window(self, sq, sk):
        """(keys before, keys after) a query may see, or None when that is all of them (full / plain causal attention)."""
        cfg = self.config
        if cfg.window_size is not None:
            pre, nxt = (x if x >= 0 else sk for x in cfg.window_size)
        elif getattr(cfg, "sparse_mode", 0) in (0, 4) and (cfg.pre_tockens != 65536 or cfg.next_tockens != 0):
            pre, nxt = cfg.pre_tockens, cfg.next_tockens          # bounds the user has set (the defaults mean "no window")
        else:
            return None
        if self.causal:
            nxt = 0
        if pre >= sk - 1 and (self.causal or nxt >= sk - 1):
            return None
        return pre, nxt

    def forward(self, q, k, v, attention_mask=None, packed_seq_params=None):
        cp = ps.get_context_parallel_world_size()
        cu = packed_seq_params.get("cu_seqlens") if isinstance(packed_seq_params, dict) else getattr(packed_seq_params, "cu_seqlens_q", None)
        win = self._window(q.shape[0] * cp, k.shape[0] * cp)
        if self.alibi_slopes is not None:
            out = self._alibi(q, k, v, cu is not None)
        elif win is not None:
            if cp > 1 or cu is not None:
                raise NotImplementedError("sliding-window attention is not combined with context parallelism or packed sequences")
            out = attn_ops.band_attention(q, k, v, win[0], win[1], softmax_scale=self.softmax_scale)
        elif cu is not None:
            # packed documents (--reset-attention-mask): every document attends to itself only
            if cp > 1:
                raise NotImplementedError("packed-sequence attention is not combined with context parallelism")
            want = getattr(self.config, "attention_backend", "auto")
            backend = "library" if want == "library" else ("sm100" if self.config.optimization_level >= 1 else None)
            out = attn_ops.varlen_attention(q, k, v, cu.tolist() if torch.is_tensor(cu) else cu, causal=self.causal,
                                            softmax_scale=self.softmax_scale, backend=backend)
        elif cp > 1:
            from ..parallel.context_parallel import dispatch_context_parallel_attention
            out = dispatch_context_parallel_attention(q, k, v, self.config, causal=self.causal,
                                                      softmax_scale=self.softmax_scale, attention_mask=attention_mask,
                                                      layer_number=self.layer_number)
        elif attention_mask is not None and not self.causal:
            out = attn_ops.attention_ref(q, k, v, causal=False, softmax_scale=self.softmax_scale, mask=attention_mask)
        else:
            # "auto": the hand-written tcgen05 forward / backward at optimisation level >= 1 (shapes it does not cover fall
            # back inside flash_attention), the library kernel at level 0; "library" / "sm100" force one
            want = getattr(self.config, "attention_backend", "auto")
            backend = None
            if want == "library":
                backend = "library"
            elif self.config.optimization_level >= 1 and want in ("auto", "sm100"):
                backend = "sm100"
            out = attn_ops.flash_attention(q, k, v, causal=self.causal, softmax_scale=self.softmax_scale, backend=backend)
        if self.dropout_p > 0 and self.training:
            with get_cuda_rng_tracker().fork():
                out = torch.nn.functional.dropout(out, self.dropout_p)
        s, b = out.shape[0], out.shape[1]
        return out.reshape(s, b, -1)


class SelfAttention(nn.Module):
    def __init__(self, config, layer_number=1, attn_mask_type="causal"):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        tp = ps.get_tensor_model_parallel_world_size()
        self.d = config.kv_channels
        self.nq_total, self.ng_total = config.num_attention_heads, config.num_query_groups
        self.nq = divide(self.nq_total, tp)
        self.ng = divide(self.ng_total, tp)
        self.qpg = self.nq // self.ng
        qkv_out = (self.nq_total + 2 * self.ng_total) * self.d
        Col, Row = linear_classes(config)
        self.linear_qkv = Col(config.hidden_size, qkv_out, config=config, init_method=config.init_method,
                                               bias=config.add_bias_linear or config.add_qkv_bias, gather_output=False,
                                               skip_bias_add=False)
        # row ranges of the q / k / v blocks inside the fused weight (per local KV group: qpg query heads, one key, one value):
        # optimizers that treat the three projections separately (Muon) read this
        blocks, row = [], 0
        for _ in range(self.ng):
            blocks.append((row, row + self.qpg * self.d)); row += self.qpg * self.d
            blocks.append((row, row + self.d)); row += self.d
            blocks.append((row, row + self.d)); row += self.d
        self.linear_qkv.weight.qkv_row_blocks = blocks
        self.core_attention = CoreAttention(config, layer_number, attn_mask_type)
        self.linear_proj = Row(self.nq_total * self.d, config.hidden_size, config=config,
                                             init_method=config.output_layer_init_method,
                                             bias=config.add_bias_linear or bool(getattr(config, "add_dense_bias", False)),
                                             input_is_parallel=True, skip_bias_add=True)
        if config.qk_layernorm:
            self.q_layernorm = build_norm(config, self.d)
            self.k_layernorm = build_norm(config, self.d)
        else:
            self.q_layernorm = self.k_layernorm = None
        self.fused_rope = config.use_fused_rotary_pos_emb or config.apply_rope_fusion or config.optimization_level >= 1

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **_):
        qkv, _ = self.linear_qkv(hidden_states)  # [s, b, ng*(qpg+2)*d]
        s, b, _w = qkv.shape
        if rotary_pos_emb is not None and self.q_layernorm is None and self.fused_rope and qkv.is_contiguous():
            cos, sin = rotary_pos_emb
            qkv = _PackedRope.apply(qkv, cos, sin, self.ng, self.qpg, self.d, self.config.rotary_interleaved)
            rotary_pos_emb = None
        v5 = qkv.view(s, b, self.ng, self.qpg + 2, self.d)
        q = _merge_group_dims(v5[:, :, :, :self.qpg])
        k = v5[:, :, :, self.qpg]
        v = v5[:, :, :, self.qpg + 1]
        if self.q_layernorm is not None:
            q, k = self.q_layernorm(q.contiguous()), self.k_layernorm(k.contiguous())
        if rotary_pos_emb is not None:
            cos, sin = rotary_pos_emb
            q = apply_rope(q, cos, sin, self.config.rotary_interleaved, fused=self.fused_rope)
            k = apply_rope(k, cos, sin, self.config.rotary_interleaved, fused=self.fused_rope)
        ctx = self.core_attention(q, k, v, attention_mask, packed_seq_params)
        return self.linear_proj(ctx)


def _merge_group_dims(q5):
    """[s,b,g,p,d] -> [s,b,g*p,d]; a view only when the (g,p) strides are mergeable, else a copy."""
    s, b, g, p, d = q5.shape
    st = q5.stride()
    if st[2] == p * st[3] or g == 1:
        return q5.as_strided((s, b, g * p, d), (st[0], st[1], st[3], st[4]), q5.storage_offset())
    return q5.reshape(s, b, g * p, d)


class MLASelfAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V2/V3): low-rank q and joint kv compression with a decoupled
    rotary key shared across heads (reference: mindspeed/core/transformer/multi_head_latent_attention/adaptor.py:23-139)."""

    def __init__(self, config, layer_number=1, attn_mask_type="causal"):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        tp = ps.get_tensor_model_parallel_world_size()
        self.n = divide(config.num_attention_heads, tp)
        self.qk_nope, self.qk_rope, self.v_dim = config.qk_head_dim, config.qk_pos_emb_head_dim, config.v_head_dim
        self.q_head_dim = self.qk_nope + self.qk_rope
        h = config.hidden_size
        from ..parallel.layers import _init_sharded  # noqa: F401
        if config.q_lora_rank is None:
            self.linear_q_proj = ColumnParallelLinear(h, config.num_attention_heads * self.q_head_dim, config=config,
                                                      init_method=config.init_method, bias=False)
        else:
            self.linear_q_down_proj = _Replicated(h, config.q_lora_rank, config)
            self.q_layernorm = build_norm(config, config.q_lora_rank)
            self.linear_q_up_proj = ColumnParallelLinear(config.q_lora_rank, config.num_attention_heads * self.q_head_dim,
                                                         config=config, init_method=config.init_method, bias=False)
        self.linear_kv_down_proj = _Replicated(h, config.kv_lora_rank + self.qk_rope, config)
        self.kv_layernorm = build_norm(config, config.kv_lora_rank)
        self.linear_kv_up_proj = ColumnParallelLinear(config.kv_lora_rank,
                                                      config.num_attention_heads * (self.qk_nope + self.v_dim),
                                                      config=config, init_method=config.init_method, bias=False)
        scale = 1.0 / math.sqrt(self.q_head_dim)
        ms = getattr(config, "mscale_all_dim", 0.0)
        if ms and getattr(config, "rotary_scaling_factor", 1) > 1:
            from .rotary import yarn_get_mscale
            m = yarn_get_mscale(config.rotary_scaling_factor, ms)
            scale = scale * m * m
        self.core_attention = CoreAttention(config, layer_number, attn_mask_type, softmax_scale=scale,
                                            k_channels=self.q_head_dim, v_channels=self.v_dim)
        self.linear_proj = RowParallelLinear(config.num_attention_heads * self.v_dim, h, config=config,
                                             init_method=config.output_layer_init_method,
                                             bias=config.add_bias_linear or bool(getattr(config, "add_dense_bias", False)),
                                             input_is_parallel=True, skip_bias_add=True)
        self.dsa = getattr(config, "experimental_attention_variant", None) == "dsa"
        if self.dsa:
            from .dsa import DSAIndexer
            if ps.get_context_parallel_world_size() > 1:
                raise NotImplementedError("DeepSeek sparse attention is not combined with context parallelism")
            self.indexer = DSAIndexer(config)

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **_):
        from ..parallel import mappings as M
        cfg = self.config
        x = hidden_states
        sp = cfg.sequence_parallel and ps.get_tensor_model_parallel_world_size() > 1
        # --recompute-mla-up-proj: the up-projections' outputs (the widest activations of the layer) are rebuilt in backward
        re_up = bool(getattr(cfg, "recompute_mla_up_proj", False)) and self.training and torch.is_grad_enabled()

        def up(lin, t):
            if re_up and t.requires_grad:
                from torch.utils.checkpoint import checkpoint
                return checkpoint(lambda z: lin(z)[0], t, use_reentrant=False)
            return lin(t)[0]
        if cfg.q_lora_rank is None:
            qc = x
            q, _ = self.linear_q_proj(x)
        else:
            qc = self.q_layernorm(self.linear_q_down_proj(x))
            q = up(self.linear_q_up_proj, qc)
        s, b = q.shape[0], q.shape[1]
        q = q.view(s, b, self.n, self.q_head_dim)
        kvc = self.linear_kv_down_proj(x)
        if sp:
            kvc = M.gather_from_sequence_parallel_region(kvc, tensor_parallel_output_grad=True)
        kv_lat, k_pe = kvc.split([cfg.kv_lora_rank, self.qk_rope], dim=-1)
        kv_lat = self.kv_layernorm(kv_lat.contiguous())
        if not self.dsa:                            # the sparse path applies the up-projection weight itself
            kv_in = M.scatter_to_sequence_parallel_region(kv_lat) if sp else kv_lat
            kv = up(self.linear_kv_up_proj, kv_in)
            kv = kv.view(s, b, self.n, self.qk_nope + self.v_dim)
            k_nope, v = kv.split([self.qk_nope, self.v_dim], dim=-1)
        q_nope, q_pe = q.split([self.qk_nope, self.qk_rope], dim=-1)
        k_pe = k_pe.reshape(s, b, 1, self.qk_rope)
        if rotary_pos_emb is not None:
            cos, sin = rotary_pos_emb
            q_pe = apply_rope(q_pe, cos, sin, cfg.rotary_interleaved, fused=False)
            k_pe = apply_rope(k_pe, cos, sin, cfg.rotary_interleaved, fused=False)
        qf = torch.cat((q_nope, q_pe), dim=-1)
        if self.dsa:
            from .dsa import dsa_attention
            xf, qcf = x.detach(), qc.detach()
            if sp:                                  # the indexer scores the whole sequence on every rank
                xf = M.gather_from_sequence_parallel_region(xf, tensor_parallel_output_grad=False)
                qcf = M.gather_from_sequence_parallel_region(qcf, tensor_parallel_output_grad=False)
            ctx = dsa_attention(self, xf, qcf, qf, kv_lat, k_pe, rotary_pos_emb)
            return self.linear_proj(ctx)
        kf = torch.cat((k_nope, k_pe.expand(s, b, self.n, self.qk_rope)), dim=-1)
        if getattr(cfg, "mla_swap_core_attn_out", False) and self.training and torch.is_grad_enabled() and qf.is_cuda:
            # --mla-swap-core-attn-out: what the attention keeps for backward (q, k, v, output, softmax statistics) waits in
            # pinned host memory
            from ..memory.host_offload import OffloadSaved
            with OffloadSaved():
                ctx = self.core_attention(qf, kf, v.contiguous(), attention_mask, packed_seq_params)
        else:
            ctx = self.core_attention(qf, kf, v.contiguous(), attention_mask, packed_seq_params)
        return self.linear_proj(ctx)


class _Replicated(nn.Module):
    """A linear whose weight is replicated across the tensor-parallel group (MLA down-projections).
    Its gradient is all-reduced over TP with the other replicated parameters when the input is sequence-sharded."""

    def __init__(self, inp, out, config):
        super().__init__()
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.empty(out, inp, device=dev, dtype=config.params_dtype))
        if config.perform_initialization:
            with torch.no_grad():
                w = torch.empty(out, inp)
                config.init_method(w)
                self.weight.copy_(w)
        setattr(self.weight, "sequence_parallel", config.sequence_parallel)

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight)
