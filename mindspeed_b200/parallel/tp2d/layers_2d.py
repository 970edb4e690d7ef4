"""Attention and MLP blocks for 2-D tensor parallelism.

Activations between blocks are [s/x, b, h/y]: the sequence split over the tp-x group, the hidden dimension over the tp-y
group.  Every block is two ``ParallelLinear2D`` with the group roles swapped, so that layout comes back after each block:

    MLP         fc1 (gather seq over x, reduce-scatter over y)  ->  [s/y, b, ffn/x]  -> activation ->
                fc2 (gather seq over y, reduce-scatter over x)  ->  [s/x, b, h/y]
    attention   qkv (x, y) -> [s/y, b, (q + 2 kv)/x]: heads split over x, sequence over y.  Rotary embedding uses the rank's
                positions; K and V are all-gathered over y along the sequence (differentiable: their gradients are
                reduce-scattered back) and the rank's query chunk attends causally to [all earlier chunks | its own chunk];
                proj (y, x) -> [s/x, b, h/y]

The sequence dimension is split contiguously (rank r of a group holds rows [r * s/n, (r + 1) * s/n)).
reference: mindspeed/core/tensor_parallel/tp_2d/parallel_linear_2d.py:24-207 (the linear), the 2-D attention / MLP wiring
of mindspeed/core/transformer/attention.py and mlp.py under --tp-2d, rotary positions per tp-y rank
(mindspeed/core/models/common/embeddings/rotary_pos_embedding.py), and the tp-y U cp grouping of
mindspeed/core/tensor_parallel_y_union_cp.py:26-99 (here K / V are gathered over tp-y; context parallelism composes on top).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import mappings as M
from .. import parallel_state as ps
from .linear_2d import ParallelLinear2D


def _size(g):
    return dist.get_world_size(g) if g is not None else 1


def _rank(g):
    return dist.get_rank(g) if g is not None else 0


class MLP2D(nn.Module):
    def __init__(self, config, gx=None, gy=None):
        super().__init__()
        self.config = config
        gx = gx if gx is not None else ps.get_tp_x_group()
        gy = gy if gy is not None else ps.get_tp_y_group()
        ffn = config.ffn_hidden_size
        self.gated = bool(config.gated_linear_unit)
        # a gated fc1 keeps gate and up projections of one slice together: each x rank owns [gate_i | up_i]
        self.linear_fc1 = ParallelLinear2D(config.hidden_size, ffn * (2 if self.gated else 1), config=config,
                                           init_method=self._gated_init(config.init_method, ffn, _size(gx)) if self.gated
                                           else config.init_method, ag_group=gx, rs_group=gy, bias=config.add_bias_linear)
        self.linear_fc2 = ParallelLinear2D(ffn, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                           ag_group=gy, rs_group=gx, bias=config.add_bias_linear)

    @staticmethod
    def _gated_init(init, ffn, nx):
        def fn(full):                      # full: [2 * ffn, h] laid out [gate | up]; reorder rows to [gate_0 | up_0 | gate_1 | ...]
            init(full)
            g, u = full[:ffn].clone(), full[ffn:].clone()
            per = ffn // nx
            for i in range(nx):
                full[2 * i * per:(2 * i + 1) * per].copy_(g[i * per:(i + 1) * per])
                full[(2 * i + 1) * per:(2 * i + 2) * per].copy_(u[i * per:(i + 1) * per])
            return full
        return fn

    def forward(self, hidden_states):
        h, _ = self.linear_fc1(hidden_states)
        if self.gated:
            g, u = h.chunk(2, dim=-1)
            a = self.config.activation_func(g) * u
        else:
            a = self.config.activation_func(h)
        return self.linear_fc2(a)


class SelfAttention2D(nn.Module):
    def __init__(self, config, layer_number=1, gx=None, gy=None):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        self.gx = gx if gx is not None else ps.get_tp_x_group()
        self.gy = gy if gy is not None else ps.get_tp_y_group()
        nx = _size(self.gx)
        self.d = config.kv_channels
        if config.num_attention_heads % nx or config.num_query_groups % nx:
            raise ValueError("2-D tensor parallel attention: heads and query groups must divide by tp-x")
        self.nq, self.ng = config.num_attention_heads // nx, config.num_query_groups // nx
        self.qpg = self.nq // self.ng
        qkv_out = (config.num_attention_heads + 2 * config.num_query_groups) * self.d
        # rows of the fused weight are grouped per KV group: [q heads of the group | k | v], so a split over x keeps whole groups
        self.linear_qkv = ParallelLinear2D(config.hidden_size, qkv_out, config=config, init_method=config.init_method,
                                           ag_group=self.gx, rs_group=self.gy, bias=config.add_bias_linear or config.add_qkv_bias)
        self.linear_proj = ParallelLinear2D(config.num_attention_heads * self.d, config.hidden_size, config=config,
                                            init_method=config.output_layer_init_method, ag_group=self.gy, rs_group=self.gx,
                                            bias=config.add_bias_linear)
        self.scale = 1.0 / (self.d ** 0.5)

    def forward(self, hidden_states, attention_mask=None, rotary_pos_emb=None, packed_seq_params=None, **_):
        from ...ops.rope import apply_rope
        from ..context_parallel.kvallgather import _PrefixCausalAttn
        qkv, _ = self.linear_qkv(hidden_states)                 # [s/y, b, ng * (qpg + 2) * d]
        s, b, _w = qkv.shape
        v5 = qkv.view(s, b, self.ng, self.qpg + 2, self.d)
        q = v5[:, :, :, :self.qpg].reshape(s, b, self.nq, self.d)
        k, v = v5[:, :, :, self.qpg], v5[:, :, :, self.qpg + 1]
        ny, ry = _size(self.gy), _rank(self.gy)
        if rotary_pos_emb is not None:
            cos, sin = rotary_pos_emb                           # rows of the full sequence: take this rank's positions
            if cos.shape[0] != s:
                cos, sin = cos[ry * s:(ry + 1) * s], sin[ry * s:(ry + 1) * s]
            q = apply_rope(q.contiguous(), cos, sin, self.config.rotary_interleaved, fused=False)
            k = apply_rope(k.contiguous(), cos, sin, self.config.rotary_interleaved, fused=False)
        k, v = k.contiguous(), v.contiguous()
        if ny > 1:
            kg = M.gather_from_sequence_parallel_region(k, tensor_parallel_output_grad=True, group=self.gy)
            vg = M.gather_from_sequence_parallel_region(v, tensor_parallel_output_grad=True, group=self.gy)
            kd, vd = kg[ry * s:(ry + 1) * s], vg[ry * s:(ry + 1) * s]
            if ry > 0:
                ctx = _PrefixCausalAttn.apply(q.contiguous(), kg[:ry * s], vg[:ry * s], kd, vd, self.scale)
            else:
                ctx = _PrefixCausalAttn.apply(q.contiguous(), None, None, kd, vd, self.scale)
        else:
            ctx = _PrefixCausalAttn.apply(q.contiguous(), None, None, k, v, self.scale)
        return self.linear_proj(ctx.reshape(s, b, self.nq * self.d))


def to_2d_layout(x, gx=None, gy=None):
    """[s, b, h] (replicated over the tensor-parallel ranks) -> this rank's [s/x, b, h/y] tile; the backward of the slice
    is the matching all-gather of the gradient tiles (sum of zero-padded tiles)."""
    gx = gx if gx is not None else ps.get_tp_x_group()
    gy = gy if gy is not None else ps.get_tp_y_group()
    return _Tile2D.apply(x, gx, gy)


def from_2d_layout(x, gx=None, gy=None):
    """[s/x, b, h/y] -> [s, b, h] on every rank (all-gather over y along the hidden dimension, over x along the sequence);
    the backward hands every rank the gradient of its tile, summed over the ranks that consumed the gathered tensor."""
    gx = gx if gx is not None else ps.get_tp_x_group()
    gy = gy if gy is not None else ps.get_tp_y_group()
    return _Untile2D.apply(x, gx, gy)


def _tile(x, gx, gy):
    x = x.chunk(_size(gx), 0)[_rank(gx)]
    return x.chunk(_size(gy), -1)[_rank(gy)].contiguous()


def _untile(x, gx, gy):
    if _size(gy) > 1:
        parts = [torch.empty_like(x) for _ in range(_size(gy))]
        dist.all_gather(parts, x.contiguous(), group=gy)
        x = torch.cat(parts, dim=-1)
    if _size(gx) > 1:
        x = M.all_gather_first_dim(x.contiguous(), gx)
    return x


class _Tile2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gx, gy):
        ctx.g = (gx, gy)
        return _tile(x, gx, gy)

    @staticmethod
    def backward(ctx, g):
        return _untile(g, *ctx.g), None, None


class _Untile2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gx, gy):
        ctx.g = (gx, gy)
        return _untile(x, gx, gy)

    @staticmethod
    def backward(ctx, g):
        gx, gy = ctx.g
        # every rank of the tensor-parallel group used the gathered tensor: the tile's gradient is the sum of their slices
        g = g.contiguous()
        for grp in (gx, gy):
            if _size(grp) > 1:
                dist.all_reduce(g, group=grp)
        return _tile(g, gx, gy), None, None
