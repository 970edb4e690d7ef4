"""Token (+ learned position) embedding with sequence-parallel scatter."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel import mappings as M
from ..parallel import parallel_state as ps
from ..parallel.layers import VocabParallelEmbedding
from ..parallel.random import get_cuda_rng_tracker


class LanguageModelEmbedding(nn.Module):
    def __init__(self, config, vocab_size, max_sequence_length, position_embedding_type="learned_absolute",
                 num_tokentypes=0, scatter_to_sequence_parallel=True):
        super().__init__()
        self.config = config
        self.add_position_embedding = position_embedding_type == "learned_absolute"
        self.scatter_to_sequence_parallel = scatter_to_sequence_parallel
        self.reduce_scatter_embeddings = (not self.add_position_embedding) and num_tokentypes <= 0 and \
            config.sequence_parallel and scatter_to_sequence_parallel and ps.get_tensor_model_parallel_world_size() > 1
        self.word_embeddings = VocabParallelEmbedding(vocab_size, config.hidden_size, init_method=config.init_method,
                                                      reduce_scatter_embeddings=self.reduce_scatter_embeddings,
                                                      config=config)
        if self.add_position_embedding:
            dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()
            self.position_embeddings = nn.Embedding(max_sequence_length, config.hidden_size, device=dev,
                                                    dtype=config.params_dtype)
            if config.perform_initialization:
                with torch.no_grad():
                    w = torch.empty(max_sequence_length, config.hidden_size)
                    config.init_method(w)
                    self.position_embeddings.weight.copy_(w)
        self.embedding_dropout = nn.Dropout(config.hidden_dropout)

    def forward(self, input_ids, position_ids, tokentype_ids=None):
        emb = self.word_embeddings(input_ids)
        if self.add_position_embedding:
            emb = emb + self.position_embeddings(position_ids)
        if not self.reduce_scatter_embeddings:
            emb = emb.transpose(0, 1).contiguous()  # [b,s,h] -> [s,b,h]
        if self.config.fp32_residual_connection:
            emb = emb.float()
        if self.config.sequence_parallel and ps.get_tensor_model_parallel_world_size() > 1:
            if not self.reduce_scatter_embeddings and self.scatter_to_sequence_parallel:
                emb = M.scatter_to_sequence_parallel_region(emb)
            if self.config.hidden_dropout > 0:
                with get_cuda_rng_tracker().fork():
                    emb = self.embedding_dropout(emb)
        elif self.config.hidden_dropout > 0:
            emb = self.embedding_dropout(emb)
        return emb
