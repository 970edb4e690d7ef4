"""DeepSeek sparse attention on top of multi-head latent attention (``--experimental-attention-variant dsa``).

A small *lightning indexer* beside every attention layer scores, for each query token, all earlier tokens
(``ops/lightning_indexer.py``); the layer then attends only to the top-k of them.  The indexer reads detached inputs and
is trained by a KL loss against the attention distribution over the selected keys, so the main model never receives
gradient through the selection.

* indexer queries come from the compressed query (``q_lora_rank`` wide), keys and per-head weights from the hidden state;
  the first ``qk_pos_emb_head_dim`` channels of both carry the rotary embedding; keys pass a LayerNorm.
* ``--use-dsa-absorb``: the query's no-position part is multiplied by the key up-projection first, so attention runs in
  the latent space against one shared row per token and only the selected rows are gathered
  (``ops/sparse_attention.sparse_latent_attention``); without it the per-head keys and values are built and the
  selection is applied to their scores.  Both give the same output.
* The KL loss is added to the backward pass through ``DSAIndexerLossScaler`` (identity on the activations) with
  ``--dsa-indexer-loss-coeff`` and the reduction of ``--kl-loss-reduction``; ``dsa_indexer_losses()`` returns the
  per-layer values of the last forward for logging.

reference: mindspeed/features_manager/transformer/experimental_attention_variant/dsa.py:5-50.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import lightning_indexer as LI
from ..ops import sparse_attention as SA
from ..ops.rope import apply_rope

_LOSSES = {}


def dsa_indexer_losses(clear: bool = False):
    """{layer number: detached indexer KL loss of the most recent forward}."""
    out = dict(_LOSSES)
    if clear:
        _LOSSES.clear()
    return out


class DSAIndexerLossScaler(torch.autograd.Function):
    """Identity on ``x``; in backward the attached loss receives ``coeff * scale`` as its gradient, where ``scale`` is
    the main loss's scale (loss scaling / micro-batch averaging), set by the schedule through ``set_loss_scale``."""
    scale = None

    @staticmethod
    def forward(ctx, x, loss, coeff):
        ctx.coeff = coeff
        ctx.save_for_backward(loss)
        return x

    @staticmethod
    def backward(ctx, g):
        (loss,) = ctx.saved_tensors
        s = DSAIndexerLossScaler.scale
        s = torch.ones((), device=loss.device) if s is None else s.to(loss.device)
        return g, torch.ones_like(loss) * s * ctx.coeff, None

    @staticmethod
    def set_loss_scale(scale):
        DSAIndexerLossScaler.scale = scale if torch.is_tensor(scale) else torch.tensor(float(scale))


class DSAIndexer(nn.Module):
    """Lightning indexer of one layer.  Parameters are replicated over tensor parallel ranks (the indexer is tiny next to
    the attention it steers); every rank scores the full sequence against the head-averaged target, so their gradients
    are identical across the group and need no reduction."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.n, self.d = config.dsa_indexer_n_heads, config.dsa_indexer_head_dim
        self.rope = config.qk_pos_emb_head_dim
        if self.rope > self.d:
            raise ValueError("--dsa-indexer-head-dim must cover the rotary channels (--qk-rope-head-dim)")
        q_in = config.q_lora_rank if config.q_lora_rank is not None else config.hidden_size
        dev = None if config.use_cpu_initialization or not torch.cuda.is_available() else torch.cuda.current_device()

        def lin(out, inp):
            w = nn.Parameter(torch.empty(out, inp, device=dev, dtype=config.params_dtype))
            if config.perform_initialization:
                with torch.no_grad():
                    t = torch.empty(out, inp)
                    config.init_method(t)
                    w.copy_(t)
            return w

        self.wq = lin(self.n * self.d, q_in)
        self.wk = lin(self.d, config.hidden_size)
        self.weights_proj = lin(self.n, config.hidden_size)
        self.k_norm = nn.LayerNorm(self.d, eps=config.layernorm_epsilon, device=dev, dtype=config.params_dtype)

    def forward(self, x, qc, rotary_pos_emb=None):
        """x [s, b, h] hidden state and qc [s, b, q_lora_rank] compressed query, both of the FULL sequence.
        Returns (indices [b, s, topk] with -1 where fewer keys are visible, scores [b, s, s])."""
        x, qc = x.detach(), qc.detach()
        s, b = x.shape[0], x.shape[1]
        q = torch.nn.functional.linear(qc, self.wq).view(s, b, self.n, self.d)
        k = self.k_norm(torch.nn.functional.linear(x, self.wk)).view(s, b, 1, self.d)
        if rotary_pos_emb is not None and self.rope:
            cos, sin = rotary_pos_emb
            il = self.config.rotary_interleaved
            q = torch.cat((apply_rope(q[..., :self.rope], cos, sin, il, fused=False), q[..., self.rope:]), dim=-1)
            k = torch.cat((apply_rope(k[..., :self.rope], cos, sin, il, fused=False), k[..., self.rope:]), dim=-1)
        w = torch.nn.functional.linear(x, self.weights_proj) * (self.n ** -0.5) * (self.d ** -0.5)     # [s, b, n]
        idx, sc = LI.indexer_topk(q.transpose(0, 1), k.squeeze(2).transpose(0, 1), w.transpose(0, 1),
                                  self.config.dsa_indexer_topk, causal=True)
        return idx, sc


def dsa_attention(self, x_full, qc_full, q, kv_lat, k_pe, rotary_pos_emb):
    """The sparse core of ``MLASelfAttention.forward``: ``q [s, b, n, dq]`` (rotary applied), ``kv_lat [s, b, r]``
    normalised latent, ``k_pe [s, b, 1, dr]`` (rotary applied).  Returns the context ``[s, b, n * dv]``."""
    cfg = self.config
    s, b = q.shape[0], q.shape[1]
    idx, sc = self.indexer(x_full, qc_full, rotary_pos_emb)
    q_nope, q_pe = q.split([self.qk_nope, self.qk_rope], dim=-1)
    scale = self.core_attention.softmax_scale
    w_up = self.linear_kv_up_proj.weight.view(self.n, self.qk_nope + self.v_dim, cfg.kv_lora_rank)
    if cfg.use_dsa_absorb:
        w_uk, w_uv = w_up[:, :self.qk_nope], w_up[:, self.qk_nope:]
        q_lat = torch.einsum("sbnd,ndr->bsnr", q_nope, w_uk.to(q.dtype))
        o_lat, p = SA.sparse_latent_attention(q_lat, q_pe.transpose(0, 1), kv_lat.transpose(0, 1),
                                              k_pe.squeeze(2).transpose(0, 1), idx, scale)
        ctx = torch.einsum("bsnr,nvr->sbnv", o_lat, w_uv.to(q.dtype))
    else:
        kv = torch.einsum("sbr,ncr->sbnc", kv_lat, w_up.to(q.dtype))
        k_nope, v = kv.split([self.qk_nope, self.v_dim], dim=-1)
        kf = torch.cat((k_nope, k_pe.expand(s, b, self.n, self.qk_rope)), dim=-1)
        o, p = SA.sparse_attention(q.transpose(0, 1), kf.transpose(0, 1), v.transpose(0, 1), idx, scale)
        ctx = o.transpose(0, 1)
    ctx = ctx.reshape(s, b, self.n * self.v_dim)
    if self.training and torch.is_grad_enabled():
        p_all = p
        from ..parallel import parallel_state as ps
        if ps.get_tensor_model_parallel_world_size() > 1:
            # heads are split over tensor-parallel ranks: the target is the mean over ALL heads
            p_all = p.detach().clone()
            torch.distributed.all_reduce(p_all, group=ps.get_tensor_model_parallel_group())
            p_all /= ps.get_tensor_model_parallel_world_size()
        loss = SA.selected_kl_loss(sc, idx, p_all, getattr(cfg, "kl_loss_reduction", "mean"))
        _LOSSES[self.layer_number] = loss.detach()
        ctx = DSAIndexerLossScaler.apply(ctx, loss, float(cfg.dsa_indexer_loss_coeff))
    return ctx
