"""Transformer layer / block.

Layer = pre-norm -> attention -> residual -> pre-norm -> MLP or MoE -> residual.
Block adds activation recompute (full: block / uniform; per-pipeline-rank counts), no-op layers for
pipeline balancing (reference: mindspeed/core/transformer/transformer_block.py:20-246,
mindspeed/core/pipeline_parallel/noop_layers/*) and the final norm.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..parallel import parallel_state as ps
from ..parallel.random import checkpoint as tp_checkpoint, get_cuda_rng_tracker, CheckpointWithoutOutput
from .attention import MLASelfAttention, SelfAttention
from .mlp import MLP
from .norms import IdentityOp, build_norm


def _bda(x, bias, residual, p, training):
    if bias is not None:
        x = x + bias
    if p > 0.0 and training:
        x = torch.nn.functional.dropout(x, p=p, training=True)
    return residual + x


class NoopTransformerLayer(nn.Module):
    """Placeholder that forwards its input; lets the layer count be padded so stages balance."""

    def __init__(self, layer_number):
        super().__init__()
        self.layer_number = layer_number

    def forward(self, hidden_states, *args, **kwargs):
        return hidden_states.clone(), None


def get_num_layers_to_build(config) -> int:
    pp = ps.get_pipeline_model_parallel_world_size()
    layout = getattr(config, "pipeline_model_parallel_layout", None)
    if layout:
        from ..parallel.pipeline.layout import PipelineLayout
        vp = ps.get_virtual_pipeline_model_parallel_rank() or 0
        return PipelineLayout.parse(layout, pp).num_decoder_layers(ps.get_pipeline_model_parallel_rank(), vp)
    per_stage = getattr(config, "pipeline_num_transformer_layers", None)
    if per_stage:
        vp = ps.get_virtual_pipeline_model_parallel_rank() or 0
        return per_stage[ps.get_pipeline_model_parallel_rank()][vp] if isinstance(per_stage[0], (list, tuple)) \
            else per_stage[ps.get_pipeline_model_parallel_rank()]
    if getattr(config, "schedules_method", None) == "dualpipev":
        return config.num_layers // pp // 2
    first, last = config.first_pipeline_num_layers, config.last_pipeline_num_layers
    if first is not None or last is not None:
        r = ps.get_pipeline_model_parallel_rank()
        middle = pp - (first is not None) - (last is not None)
        rest = config.num_layers - (first or 0) - (last or 0)
        if r == 0 and first is not None:
            n = first
        elif r == pp - 1 and last is not None:
            n = last
        else:
            n = rest // max(middle, 1)
    else:
        n = config.num_layers // pp
    vpp = ps.get_virtual_pipeline_model_parallel_world_size()
    if vpp is not None:
        n //= vpp
    return n


def get_transformer_layer_offset(config, vp_stage: Optional[int] = None) -> int:
    pp = ps.get_pipeline_model_parallel_world_size()
    r = ps.get_pipeline_model_parallel_rank()
    layout = getattr(config, "pipeline_model_parallel_layout", None)
    if layout:
        from ..parallel.pipeline.layout import PipelineLayout
        vp = vp_stage if vp_stage is not None else (ps.get_virtual_pipeline_model_parallel_rank() or 0)
        return PipelineLayout.parse(layout, pp).layer_offset(r, vp)
    if getattr(config, "schedules_method", None) == "dualpipev":
        per = config.num_layers // pp // 2
        chunk = vp_stage if vp_stage is not None else (ps.get_virtual_pipeline_model_parallel_rank() or 0)
        # chunk 0 holds layers [r*per, ...), chunk 1 holds the mirror slice counted from the end
        # (reference: mindspeed/core/pipeline_parallel/dualpipev/dualpipev_chunks.py:43-53)
        return r * per if chunk == 0 else config.num_layers - (r + 1) * per
    per_stage = getattr(config, "pipeline_num_transformer_layers", None)
    if per_stage:
        # explicit (possibly uneven) layer counts: the offset is what the stages before this one hold
        if isinstance(per_stage[0], (list, tuple)):
            vp = vp_stage if vp_stage is not None else (ps.get_virtual_pipeline_model_parallel_rank() or 0)
            before = sum(per_stage[rr][v] for v in range(vp) for rr in range(pp))
            return before + sum(per_stage[rr][vp] for rr in range(r))
        return sum(per_stage[:r])
    n = get_num_layers_to_build(config)
    vpp = ps.get_virtual_pipeline_model_parallel_world_size()
    if vpp is not None:
        vp = vp_stage if vp_stage is not None else ps.get_virtual_pipeline_model_parallel_rank()
        total_per_vp = config.num_layers // vpp
        return vp * total_per_vp + r * n
    first = config.first_pipeline_num_layers
    if first is not None and r > 0:
        return first + (r - 1) * n
    return r * n


class TransformerLayer(nn.Module):
    def __init__(self, config, layer_number=1, hidden_dropout=None, is_moe=None):
        super().__init__()
        self.config = config
        self.layer_number = layer_number + get_transformer_layer_offset(config)
        self.hidden_dropout = config.hidden_dropout if hidden_dropout is None else hidden_dropout
        self.input_layernorm = build_norm(config, config.hidden_size)
        tp2d = bool(getattr(config, "tp_2d", False))
        if tp2d:
            # 2-D tensor parallelism: activations between blocks are [s/x, b, h/y] (parallel/tp2d/layers_2d.py)
            if config.multi_latent_attention or getattr(config, "attention_mask_type", "causal") != "causal":
                raise NotImplementedError("--tp-2d supports causal multi-head / grouped-query attention")
            from ..parallel.tp2d import MLP2D, SelfAttention2D
            self.self_attention = SelfAttention2D(config, self.layer_number)
        else:
            attn_cls = MLASelfAttention if config.multi_latent_attention else SelfAttention
            self.self_attention = attn_cls(config, self.layer_number, attn_mask_type=getattr(config, "attention_mask_type", "causal"))
        self.pre_mlp_layernorm = build_norm(config, config.hidden_size)
        if is_moe is None:
            is_moe = _is_moe_layer(config, self.layer_number)
        self.is_moe = is_moe
        self.ampipe, self._ampipe_streams = 1, None      # > 1 only with the DeepSpeed-style MoE (set below)
        if is_moe and getattr(config, "moe_model_type", "megatron_moe") == "deepspeed_moe":
            from ..legacy_moe.adapter import LegacyMoEBlock
            self.mlp = LegacyMoEBlock(config, layer_number=self.layer_number)
            self.ampipe = int(getattr(config, "ampipe_degree", 1) or 1)
        elif is_moe:
            from ..parallel.moe.moe_layer import MoELayer
            self.mlp = MoELayer(config, layer_number=self.layer_number)
        elif tp2d:
            self.mlp = MLP2D(config)
        else:
            self.mlp = MLP(config)
        # --recompute-module-list with --recompute-type 0 / 1: the first N layers of this pipeline rank recompute only their
        # MLP block / attention block in backward (reference: the module-level policy of mindspeed/core/memory/auto_pipeline)
        rml, rtype = getattr(config, "recompute_module_list", None), getattr(config, "recompute_type", 2)
        n_blk = rml[ps.get_pipeline_model_parallel_rank()] if isinstance(rml, (list, tuple)) and rtype in (0, 1) else 0
        plain_residual = not config.apply_residual_connection_post_layernorm      # the block's norm lives inside the checkpoint
        self.recompute_mlp_block = rtype == 0 and layer_number <= n_blk and plain_residual
        self.recompute_attn_block = rtype == 1 and layer_number <= n_blk and plain_residual
        sel = getattr(config, "compress_activation", None) or []
        self.compress_saved = isinstance(sel, (list, tuple)) and self.layer_number in sel
        self.recompute_norm = bool(getattr(config, "recompute_norm", False))
        # --recompute-norm-num-layers / --recompute-activation-function-num-layers: only the first N layers of a stage
        n_norm = getattr(config, "recompute_norm_num_layers", None)
        if n_norm is not None and layer_number > n_norm:
            self.recompute_norm = False
        n_act = getattr(config, "recompute_activation_function_num_layers", None)
        if n_act is not None and layer_number > n_act and hasattr(self.mlp, "recompute_activation"):
            self.mlp.recompute_activation = False

    def _norm(self, norm, x):
        return norm(x)

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **kwargs):
        if self.compress_saved and self.training and torch.is_grad_enabled():
            # --compress-activation: what this layer saves for backward is stored losslessly compressed
            from ..memory.compress_activation import CompressSavedActivations
            with CompressSavedActivations():
                return self._forward(hidden_states, attention_mask, rotary_pos_emb, packed_seq_params, **kwargs)
        return self._forward(hidden_states, attention_mask, rotary_pos_emb, packed_seq_params, **kwargs)

    def _ampipe_tail(self, attn_out, attn_bias, residual):
        """``--ampipe-degree d``: everything behind the attention - residual add, norm, the DeepSpeed-style MoE, residual add -
        runs on d slices of the sequence, slice after slice, each MoE on one of two side streams: while slice i's tokens are
        exchanged and run through their experts, slice i + 1 is already normalised, gated and dispatched, so all-to-alls of
        one slice overlap expert GEMMs of the other.  Every slice is routed on its own (capacity per slice).
        reference: the ampipe option of the DeepSpeed-style MoE (mindspeed/arguments.py:336-340, 803-820; mindspeed/moe/utils.py:73-102
        slice index helpers)."""
        d = self.ampipe
        s = attn_out.shape[0]
        if s % d != 0:
            raise ValueError(f"--ampipe-degree {d} must divide the local sequence length {s}")
        use_streams = attn_out.is_cuda
        if use_streams and self._ampipe_streams is None:
            self._ampipe_streams = (torch.cuda.Stream(), torch.cuda.Stream())
        main = torch.cuda.current_stream() if use_streams else None
        outs = []
        for i, (a, r) in enumerate(zip(attn_out.chunk(d, dim=0), residual.chunk(d, dim=0))):
            h = _bda(a, attn_bias, r, self.hidden_dropout, self.training)
            x = self.pre_mlp_layernorm(h)
            if use_streams:
                side = self._ampipe_streams[i % 2]
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    m, mb = self.mlp(x)
                    o = _bda(m, mb, x if self.config.apply_residual_connection_post_layernorm else h, self.hidden_dropout, self.training)
                x.record_stream(side)                 # made on the main stream, read on the side stream ...
                h.record_stream(side)
                o.record_stream(main)                 # ... and the other way round
            else:
                m, mb = self.mlp(x)
                o = _bda(m, mb, x if self.config.apply_residual_connection_post_layernorm else h, self.hidden_dropout, self.training)
            outs.append(o)
        if use_streams:
            for side in self._ampipe_streams:
                main.wait_stream(side)
        return torch.cat(outs, dim=0)

    def _forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **kwargs):
        residual = hidden_states
        if self.recompute_norm and self.training and hidden_states.requires_grad:
            ck = CheckpointWithoutOutput()
            ln = ck.checkpoint(self.input_layernorm, False, hidden_states)
            attn_out, attn_bias = self.self_attention(ln, attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                                      packed_seq_params=packed_seq_params)
            ck.discard_output()
            attn_out.register_hook(ck.recompute)
        elif self.recompute_attn_block and self.training and hidden_states.requires_grad:
            from ..parallel.random import checkpoint

            def attn_block(h):
                o, b_ = self.self_attention(self.input_layernorm(h), attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                            packed_seq_params=packed_seq_params)
                return o if b_ is None else o + b_
            ln = None
            attn_out, attn_bias = checkpoint(attn_block, False, hidden_states), None
        else:
            ln = self.input_layernorm(hidden_states)
            attn_out, attn_bias = self.self_attention(ln, attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                                      packed_seq_params=packed_seq_params)
        if self.config.apply_residual_connection_post_layernorm:
            residual = ln
        if self.ampipe > 1:
            return self._ampipe_tail(attn_out, attn_bias, residual), None
        ln2 = None
        if (attn_bias is None and not (self.hidden_dropout > 0.0 and self.training) and not self.recompute_norm
                and not self.recompute_mlp_block and not self.config.apply_residual_connection_post_layernorm and hasattr(self.pre_mlp_layernorm, "forward_add")):
            # residual add and the MLP's norm in one pass over the row (and one kernel in backward)
            hidden_states, ln2 = self.pre_mlp_layernorm.forward_add(attn_out, residual)
        else:
            hidden_states = _bda(attn_out, attn_bias, residual, self.hidden_dropout, self.training)
        residual = hidden_states
        if self.recompute_mlp_block and self.training and hidden_states.requires_grad and not self.is_moe:
            from ..parallel.random import checkpoint

            def mlp_block(h):
                o, b_ = self.mlp(self.pre_mlp_layernorm(h))
                return o if b_ is None else o + b_
            mlp_out, mlp_bias = checkpoint(mlp_block, False, hidden_states), None
        elif ln2 is not None:
            mlp_out, mlp_bias = self.mlp(ln2)
        elif self.recompute_norm and self.training and hidden_states.requires_grad and not self.is_moe:
            ck2 = CheckpointWithoutOutput()
            ln2 = ck2.checkpoint(self.pre_mlp_layernorm, False, hidden_states)
            mlp_out, mlp_bias = self.mlp(ln2)
            ck2.discard_output()
            mlp_out.register_hook(ck2.recompute)
        else:
            ln2 = self.pre_mlp_layernorm(hidden_states)
            mlp_out, mlp_bias = self.mlp(ln2)
        if self.config.apply_residual_connection_post_layernorm:
            residual = ln2
        hidden_states = _bda(mlp_out, mlp_bias, residual, self.hidden_dropout, self.training)
        return hidden_states, None


def _is_moe_layer(config, layer_number) -> bool:
    if config.num_moe_experts is None:
        return False
    if layer_number <= getattr(config, "first_k_dense_replace", 0):
        return False
    freq = config.moe_layer_freq
    if isinstance(freq, int):
        return (layer_number - 1) % freq == 0 if freq > 1 else True
    return bool(freq[layer_number - 1])


class TransformerBlock(nn.Module):
    def __init__(self, config, pre_process=True, post_process=True, post_layer_norm=True, vp_stage=None):
        super().__init__()
        self.config, self.pre_process, self.post_process = config, pre_process, post_process
        self.input_tensor = None
        n = get_num_layers_to_build(config)
        offset = get_transformer_layer_offset(config, vp_stage)
        noop = set(getattr(config, "noop_layers", None) or [])
        layers = []
        for i in range(n):
            if (offset + i) in noop:
                layers.append(NoopTransformerLayer(offset + i + 1))
            else:
                layers.append(TransformerLayer(config, layer_number=i + 1))
        self.layers = nn.ModuleList(layers)
        self.num_layers_per_pipeline_rank = n
        self.fb_state, self.fb_partner = None, None      # pipeline schedules: parallel/moe/fb_overlap.StagedBlockState
        self.fb_overlap = None           # set by the schedule for the duration of one step (parallel/moe/fb_overlap.BlockOverlap)
        self.final_layernorm = build_norm(config, config.hidden_size) if (post_process and post_layer_norm) else None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def _recompute_count(self):
        cfg = self.config
        n = cfg.recompute_num_layers
        if getattr(cfg, "enable_recompute_layers_per_pp_rank", False) and isinstance(n, (list, tuple)):
            # per pipeline rank (and virtual stage) layer counts
            # (reference: mindspeed/core/transformer/transformer_block.py:20-156)
            vp = ps.get_virtual_pipeline_model_parallel_rank() or 0
            n = n[ps.get_pipeline_model_parallel_rank()]
            if isinstance(n, (list, tuple)):
                n = n[vp]
        return n

    def _checkpointed_forward(self, hidden_states, attention_mask, rotary_pos_emb, packed_seq_params):
        def custom(start, end):
            def run(h, mask, cos, sin):
                rpe = None if cos is None else (cos, sin)
                for i in range(start, end):
                    h, _ = self.layers[i](h, attention_mask=mask, rotary_pos_emb=rpe, packed_seq_params=packed_seq_params)
                return h
            return run
        cos, sin = (None, None) if rotary_pos_emb is None else rotary_pos_emb
        n = len(self.layers)
        cnt = self._recompute_count()
        if self.config.recompute_method == "uniform":
            i = 0
            while i < n:
                j = min(i + cnt, n)
                hidden_states = tp_checkpoint(custom(i, j), self.config.distribute_saved_activations, hidden_states,
                                              attention_mask, cos, sin)
                i = j
        else:  # block: checkpoint the first `cnt` real layers, run the rest normally
            done = 0
            for i in range(n):
                is_noop = isinstance(self.layers[i], NoopTransformerLayer)
                if done < cnt and not is_noop:
                    hidden_states = tp_checkpoint(custom(i, i + 1), self.config.distribute_saved_activations,
                                                  hidden_states, attention_mask, cos, sin)
                    done += 1
                else:
                    hidden_states = custom(i, i + 1)(hidden_states, attention_mask, cos, sin)
        return hidden_states

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **kwargs):
        if not self.pre_process:
            hidden_states = self.input_tensor
        tp2d = bool(getattr(self.config, "tp_2d", False))
        if tp2d and self.pre_process:
            from ..parallel.tp2d import to_2d_layout
            hidden_states = to_2d_layout(hidden_states)          # [s, b, h] from the embedding -> this rank's [s/x, b, h/y]
        if self.fb_state is not None and self.training and torch.is_grad_enabled():
            # pipeline form of --moe-fb-overlap: staged graphs per (chunk, micro-batch); a partner's backward may ride along
            from ..parallel.pipeline.executor import current_microbatch
            cur = current_microbatch()
            hidden_states = self.fb_state.forward((cur["chunk"], cur["mb"]), hidden_states, partner=self.fb_partner,
                                                  attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                                  packed_seq_params=packed_seq_params)
        elif self.fb_overlap is not None and self.training and torch.is_grad_enabled():
            # forward of this micro-batch interleaved with the layer backward of the previous one (--moe-fb-overlap);
            # returns a detached leaf: the schedule's loss backward stops there and seeds the next interleaved backward
            hidden_states = self.fb_overlap.forward(hidden_states, attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                                    packed_seq_params=packed_seq_params)
        elif self.config.recompute_granularity == "full" and self.training:
            hidden_states = self._checkpointed_forward(hidden_states, attention_mask, rotary_pos_emb, packed_seq_params)
        else:
            for layer in self.layers:
                hidden_states, _ = layer(hidden_states, attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb,
                                         packed_seq_params=packed_seq_params)
        if self.final_layernorm is not None:
            hidden_states = self.final_layernorm(hidden_states)
        if tp2d and self.post_process:
            from ..parallel.tp2d import from_2d_layout
            hidden_states = from_2d_layout(hidden_states)        # back to [s, b, h] for the output layer
        return hidden_states
