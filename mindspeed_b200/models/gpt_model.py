"""GPT decoder language model (Megatron-core ``GPTModel`` surface).

forward(input_ids, position_ids, attention_mask, labels) -> per-token loss [b, s] when labels are
given on the last pipeline stage, else logits [b, s, V/tp] or hidden states for the next stage.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..parallel import mappings as M
from ..parallel import parallel_state as ps
from ..parallel.cross_entropy import vocab_parallel_cross_entropy
from ..parallel.layers import ColumnParallelLinear
from .embedding import LanguageModelEmbedding
from .rotary import RotaryEmbedding, cp_local_positions
from .transformer import TransformerBlock


class GPTModel(nn.Module):
    def __init__(self, config, transformer_layer_spec=None, vocab_size: int = 0, max_sequence_length: int = 0,
                 pre_process: bool = True, post_process: bool = True, fp16_lm_cross_entropy: bool = False,
                 parallel_output: bool = True, share_embeddings_and_output_weights: bool = False,
                 position_embedding_type: str = "learned_absolute", rotary_percent: float = 1.0,
                 rotary_base: int = 10000, rope_scaling: bool = False, rope_scaling_factor: float = 8.0,
                 scatter_embedding_sequence_parallel: bool = True, seq_len_interpolation_factor: Optional[float] = None,
                 mtp_block_spec=None, vp_stage: Optional[int] = None):
        super().__init__()
        self.config = config
        self.vocab_size, self.max_sequence_length = vocab_size, max_sequence_length
        self.pre_process, self.post_process = pre_process, post_process
        self.parallel_output = parallel_output
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        self.position_embedding_type = position_embedding_type
        if position_embedding_type == "alibi":
            config.position_embedding_type = "alibi"            # read by the attention layers (bias from head slopes)
        self.fp16_lm_cross_entropy = fp16_lm_cross_entropy
        self.vp_stage = vp_stage
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type,
                                                    scatter_to_sequence_parallel=scatter_embedding_sequence_parallel)
        if position_embedding_type in ("rope", "yarn"):
            if config.multi_latent_attention:
                yarn = None
                if getattr(config, "rope_type", "rope") == "yarn" and getattr(config, "rotary_scaling_factor", 1) > 1:
                    yarn = dict(factor=config.rotary_scaling_factor,
                                original_max_position_embeddings=config.original_max_position_embeddings,
                                beta_fast=config.beta_fast, beta_slow=config.beta_slow, mscale=config.mscale,
                                mscale_all_dim=config.mscale_all_dim)
                self.rotary_pos_emb = RotaryEmbedding(config.qk_pos_emb_head_dim, 1.0, config.rotary_interleaved,
                                                      seq_len_interpolation_factor, getattr(config, "rotary_base", rotary_base),
                                                      yarn=yarn)
            else:
                self.rotary_pos_emb = RotaryEmbedding(config.kv_channels, rotary_percent, config.rotary_interleaved,
                                                      seq_len_interpolation_factor, rotary_base, rope_scaling,
                                                      rope_scaling_factor)
        else:
            self.rotary_pos_emb = None
        self.decoder = TransformerBlock(config, pre_process=pre_process, post_process=post_process, vp_stage=vp_stage)
        if post_process:
            skip = pre_process and share_embeddings_and_output_weights
            self.output_layer = ColumnParallelLinear(config.hidden_size, vocab_size, config=config,
                                                     init_method=config.init_method, bias=False, gather_output=not parallel_output,
                                                     skip_bias_add=False, skip_weight_param_allocation=skip)
            if share_embeddings_and_output_weights and not skip:
                self.output_layer.weight.data.zero_()
                self.output_layer.weight.shared_embedding = True
        if pre_process and share_embeddings_and_output_weights:
            self.embedding.word_embeddings.weight.shared_embedding = True
        self.mtp = None
        if getattr(config, "mtp_num_layers", None) and post_process:
            from .mtp import MultiTokenPredictionBlock
            self.mtp = MultiTokenPredictionBlock(config, vocab_size)

    def set_input_tensor(self, input_tensor):
        if isinstance(input_tensor, (list, tuple)):
            input_tensor = input_tensor[0]
        self.decoder.set_input_tensor(input_tensor)

    def shared_embedding_or_output_weight(self):
        if self.pre_process:
            return self.embedding.word_embeddings.weight
        if self.post_process:
            return self.output_layer.weight
        return None

    def _rotary(self, seq_len_local, device):
        if self.rotary_pos_emb is None:
            return None
        cfg = self.config
        cp = ps.get_context_parallel_world_size()
        full = seq_len_local * cp
        if cp > 1:
            pos = cp_local_positions(full, cp, ps.get_context_parallel_rank(),
                                     getattr(cfg, "context_parallel_algo", "megatron_cp_algo"), device=device)
            if getattr(cfg, "context_parallel_algo", "") == "hybrid_cp_algo":
                from ..parallel.context_parallel.batch_utils import hybrid_local_positions
                pos = hybrid_local_positions(full, device)
            return self.rotary_pos_emb.get_cos_sin(full, device, positions=pos)
        return self.rotary_pos_emb.get_cos_sin(full, device)

    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_params=None, packed_seq_params=None, extra_block_kwargs=None, loss_mask=None, **_):
        if decoder_input is None and self.pre_process:
            decoder_input = self.embedding(input_ids, position_ids)
        if self.pre_process:
            s_local = input_ids.shape[1]
            dev = input_ids.device
        else:
            inp = self.decoder.input_tensor
            s_local = inp.shape[0] * (ps.get_tensor_model_parallel_world_size() if self.config.sequence_parallel else 1)
            dev = inp.device
        rpe = self._rotary(s_local, dev)
        pos_reset = packed_seq_params.get("position_ids") if isinstance(packed_seq_params, dict) else None
        if pos_reset is not None and self.rotary_pos_emb is not None:
            # positions restart at every document (--reset-position-ids): the rotary angles follow them
            if pos_reset.dim() == 2 and pos_reset.shape[0] != 1:
                raise NotImplementedError("per-document rotary positions take micro-batch size 1")
            rpe = self.rotary_pos_emb.get_cos_sin(s_local, dev, positions=pos_reset.reshape(-1).to(dev))
        hidden = self.decoder(decoder_input, attention_mask=attention_mask, rotary_pos_emb=rpe,
                              packed_seq_params=packed_seq_params)
        if not self.post_process:
            return hidden
        weight = self.shared_embedding_or_output_weight() if self.share_embeddings_and_output_weights else None
        mtp_loss = None
        if self.mtp is not None and labels is not None and self.training:
            mtp_loss = self.mtp(hidden, input_ids, position_ids, labels, loss_mask, self, rpe, attention_mask)
        logits, _ = self.output_layer(hidden, weight=weight)  # [s, b, V/tp]
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        loss = self.compute_language_model_loss(labels, logits)
        if mtp_loss is not None:
            loss = loss + mtp_loss
        return loss

    def compute_language_model_loss(self, labels, logits):
        labels_sb = labels.transpose(0, 1).contiguous()  # [s, b]
        if self.fp16_lm_cross_entropy or logits.is_cuda:
            loss = vocab_parallel_cross_entropy(logits, labels_sb)
        else:
            loss = vocab_parallel_cross_entropy(logits.float(), labels_sb)
        return loss.transpose(0, 1).contiguous()  # [b, s]

    def sharded_state_dict(self, prefix="", sharded_offsets=(), metadata=None):
        from ..checkpointing.sharded import model_sharded_state_dict
        return model_sharded_state_dict(self, prefix)
