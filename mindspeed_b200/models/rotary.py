"""Rotary embeddings: plain, linear-scaled and YaRN
(reference: mindspeed/core/models/common/embeddings/rotary_pos_embedding.py:28-114)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..parallel import parallel_state as ps


def _yarn_find_correction_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_find_correction_range(low_rot, high_rot, dim, base, max_pos):
    low = math.floor(_yarn_find_correction_dim(low_rot, dim, base, max_pos))
    high = math.ceil(_yarn_find_correction_dim(high_rot, dim, base, max_pos))
    return max(low, 0), min(high, dim - 1)


def yarn_get_mscale(scale=1.0, mscale=1.0):
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class RotaryEmbedding(nn.Module):
    def __init__(self, kv_channels, rotary_percent=1.0, rotary_interleaved=False, seq_len_interpolation_factor=None,
                 rotary_base=10000, rope_scaling=False, rope_scaling_factor=8.0, use_cpu_initialization=False,
                 yarn=None):
        super().__init__()
        dim = kv_channels if rotary_percent >= 1.0 else int(kv_channels * rotary_percent)
        self.dim, self.rotary_interleaved = dim, rotary_interleaved
        self.seq_len_interpolation_factor = seq_len_interpolation_factor
        inv_freq = 1.0 / (rotary_base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.mscale = 1.0
        if rope_scaling:  # llama-3.1 style frequency-dependent scaling
            inv_freq = self._llama3_scale(inv_freq, rope_scaling_factor)
        if yarn is not None:
            # yarn = dict(factor, original_max_position_embeddings, beta_fast, beta_slow, mscale, mscale_all_dim)
            f, orig = yarn["factor"], yarn["original_max_position_embeddings"]
            lo, hi = _yarn_find_correction_range(yarn.get("beta_fast", 32), yarn.get("beta_slow", 1), dim, rotary_base, orig)
            ramp = ((torch.arange(dim // 2, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            mask = 1.0 - ramp
            inv_freq = inv_freq / f * (1 - mask) + inv_freq * mask
            self.mscale = yarn_get_mscale(f, yarn.get("mscale", 1.0)) / yarn_get_mscale(f, yarn.get("mscale_all_dim", 0.0) or 1.0) \
                if yarn.get("mscale_all_dim", 0.0) else yarn_get_mscale(f, yarn.get("mscale", 1.0))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._cache = {}

    @staticmethod
    def _llama3_scale(inv_freq, factor, low_freq_factor=1.0, high_freq_factor=4.0, original=8192):
        wavelen = 2 * math.pi / inv_freq
        low_w, high_w = original / low_freq_factor, original / high_freq_factor
        smooth = ((original / wavelen) - low_freq_factor) / (high_freq_factor - low_freq_factor)
        scaled = torch.where(wavelen > low_w, inv_freq / factor, inv_freq)
        mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
        return torch.where((wavelen <= low_w) & (wavelen >= high_w), mid, scaled)

    def get_cos_sin(self, max_seq_len, device, positions=None, offset=0):
        """cos, sin fp32 [len, dim]; with context parallelism pass the local absolute ``positions``."""
        key = (max_seq_len, str(device), offset, None if positions is None else (positions.data_ptr(), positions.numel()))
        if positions is None and key in self._cache:
            return self._cache[key]
        pos = positions.float().to(device) if positions is not None else \
            torch.arange(max_seq_len, dtype=torch.float32, device=device) + offset
        if self.seq_len_interpolation_factor is not None:
            pos = pos / self.seq_len_interpolation_factor
        freqs = torch.outer(pos, self.inv_freq.to(device))
        if self.rotary_interleaved:
            emb = torch.stack((freqs, freqs), dim=-1).reshape(freqs.shape[0], -1)
        else:
            emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = (emb.cos() * self.mscale).contiguous(), (emb.sin() * self.mscale).contiguous()
        if positions is None:
            self._cache[key] = (cos, sin)
        return cos, sin

    def forward(self, max_seq_len, offset=0, packed_seq=False):
        """Megatron-compatible: raw angles [s, 1, 1, dim]."""
        pos = torch.arange(max_seq_len, dtype=torch.float32, device=self.inv_freq.device) + offset
        freqs = torch.outer(pos, self.inv_freq)
        emb = torch.cat((freqs, freqs), dim=-1) if not self.rotary_interleaved else \
            torch.stack((freqs, freqs), dim=-1).reshape(freqs.shape[0], -1)
        emb = emb[:, None, None, :]
        if ps.get_context_parallel_world_size() > 1 and not packed_seq:
            emb = get_pos_emb_on_this_cp_rank(emb, 0)
        return emb

    def get_rotary_seq_len(self, inference_params, transformer, transformer_input, transformer_config, packed_seq_params=None):
        if transformer_input is not None:
            n = transformer_input.size(0)
        else:
            n = transformer.input_tensor.size(0)
        if transformer_config.sequence_parallel:
            n *= transformer_config.tensor_model_parallel_size
        return n * transformer_config.context_parallel_size


def cp_local_positions(seq_len, cp_size, cp_rank, algo="megatron_cp_algo", device=None):
    """Absolute positions of the tokens this context-parallel rank holds.
    Ring attention uses the causal load-balanced split (chunks r and 2cp-1-r of 2cp); Ulysses and
    KV-allgather keep contiguous chunks (reference: mindspeed/core/context_parallel/get_batch_utils.py:244-277)."""
    if cp_size == 1:
        return torch.arange(seq_len, device=device)
    if algo in ("ulysses_cp_algo",):
        per = seq_len // cp_size
        return torch.arange(cp_rank * per, (cp_rank + 1) * per, device=device)
    per = seq_len // (2 * cp_size)
    a = torch.arange(cp_rank * per, (cp_rank + 1) * per, device=device)
    j = 2 * cp_size - 1 - cp_rank
    b = torch.arange(j * per, (j + 1) * per, device=device)
    return torch.cat((a, b))


def get_pos_emb_on_this_cp_rank(pos_emb, seq_dim):
    cp, r = ps.get_context_parallel_world_size(), ps.get_context_parallel_rank()
    idx = cp_local_positions(pos_emb.shape[seq_dim], cp, r, device=pos_emb.device)
    return pos_emb.index_select(seq_dim, idx)
