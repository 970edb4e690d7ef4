"""Multi-token prediction (DeepSeek-V3): depth k predicts token t+1+k from the main model's hidden state at t combined
with the embedding of token t+k:   h_k = Layer_k( W_k [RMSNorm(h_{k-1}) ; RMSNorm(Emb(x_{t+k}))] ),  shared output head.
The depth losses are averaged and scaled by ``mtp_loss_scaling_factor``
(Megatron-core ``MultiTokenPredictionBlock`` surface; DualPipeV handling in the reference:
mindspeed/core/pipeline_parallel/dualpipev/mtp_utils.py)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel.cross_entropy import vocab_parallel_cross_entropy
from .norms import build_norm


def _roll_left(t, k, dim=1, fill=0):
    out = torch.roll(t, shifts=-k, dims=dim)
    idx = [slice(None)] * t.dim()
    idx[dim] = slice(t.shape[dim] - k, None)
    out[tuple(idx)] = fill
    return out


class MultiTokenPredictionLayer(nn.Module):
    def __init__(self, config, layer_number):
        super().__init__()
        from .transformer import TransformerLayer
        self.enorm = build_norm(config, config.hidden_size)
        self.hnorm = build_norm(config, config.hidden_size)
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
        self.eh_proj = nn.Linear(2 * config.hidden_size, config.hidden_size, bias=False, device=dev, dtype=config.params_dtype)
        with torch.no_grad():
            config.init_method(self.eh_proj.weight)
        self.transformer_layer = TransformerLayer(config, layer_number=layer_number, is_moe=False)
        self.final_layernorm = build_norm(config, config.hidden_size)

    def forward(self, hidden, emb, rotary_pos_emb, attention_mask):
        x = self.eh_proj(torch.cat((self.enorm(emb), self.hnorm(hidden)), dim=-1))
        x, _ = self.transformer_layer(x, attention_mask=attention_mask, rotary_pos_emb=rotary_pos_emb)
        return self.final_layernorm(x)


class MultiTokenPredictionBlock(nn.Module):
    def __init__(self, config, vocab_size):
        super().__init__()
        if config.sequence_parallel and config.tensor_model_parallel_size > 1:
            raise NotImplementedError("multi-token prediction runs on unsharded sequences; disable sequence parallel for it")
        self.config = config
        self.layers = nn.ModuleList([MultiTokenPredictionLayer(config, config.num_layers + 1 + i) for i in range(config.mtp_num_layers)])
        self.scale = config.mtp_loss_scaling_factor if config.mtp_loss_scaling_factor is not None else 0.1

    def forward(self, hidden, input_ids, position_ids, labels, loss_mask, model, rotary_pos_emb, attention_mask):
        """hidden [s, b, h] from the main decoder (after its final norm).  Returns the scaled MTP loss [b, s]."""
        total = None
        ids, lab = input_ids, labels
        h = hidden
        for k, layer in enumerate(self.layers):
            ids, lab = _roll_left(ids, 1), _roll_left(lab, 1)
            if model.pre_process:
                emb = model.embedding(ids, position_ids)
            else:
                raise NotImplementedError("MTP needs the embedding on the loss stage (DualPipeV places both on rank 0)")
            h = layer(h, emb, rotary_pos_emb, attention_mask)
            weight = model.shared_embedding_or_output_weight() if model.share_embeddings_and_output_weights else None
            logits, _ = model.output_layer(h, weight=weight)
            loss = vocab_parallel_cross_entropy(logits if logits.is_cuda else logits.float(), lab.transpose(0, 1).contiguous()).transpose(0, 1)
            valid = torch.ones_like(loss)
            valid[:, loss.shape[1] - (k + 1):] = 0          # the last k+1 positions have no target
            loss = loss * valid
            total = loss if total is None else total + loss
        return total * (self.scale / len(self.layers))
