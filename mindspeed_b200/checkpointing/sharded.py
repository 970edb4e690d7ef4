"""Sharded-tensor descriptions of model and optimizer state (the ``torch_dist`` checkpoint layout).

A ``ShardedTensor`` names a global tensor (``key``, ``global_shape``) and says which rectangular chunk of it the
local data is (``global_offset``); ``replica_id`` 0 marks the copy that gets written when several ranks hold the
same chunk.  Saving turns each into one shard write item of ``torch.distributed.checkpoint``, which writes ``.metadata`` +
``__{rank}_{n}.distcp``; loading under a different tensor / pipeline / data-parallel layout re-reads whichever chunks
overlap the new local shards.  Per-layer tensors are stacked along a leading layer axis under a key without the layer
number, as Megatron-core does.
(Megatron-core ``dist_checkpointing`` surface; reference usage mindspeed/checkpointing.py:78-106.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parallel import parallel_state as ps


@dataclass
class ShardedTensor:
    key: str
    data: torch.Tensor
    global_shape: Tuple[int, ...]
    global_offset: Tuple[int, ...]
    replica_id: int = 0

    @property
    def local_shape(self):
        return tuple(self.data.shape)


def make_tp_sharded_tensors(state_dict: Dict[str, torch.Tensor], prefix: str, tp_axis_map: Dict[str, int], sharded_offsets=(),
                            tp_rank: int = 0, tp_world: int = 1, extra_replica: int = 0) -> Dict[str, ShardedTensor]:
    """``tp_axis_map``: parameter name -> axis split over tensor parallel ranks; anything else is replicated."""
    out = {}
    dp_rank = ps.get_data_parallel_rank(with_context_parallel=True) if ps.model_parallel_is_initialized() else 0
    for name, t in state_dict.items():
        if t is None or not torch.is_tensor(t):
            continue
        key = f"{prefix}{name}"
        if name in tp_axis_map and tp_world > 1:
            ax = tp_axis_map[name]
            gshape = list(t.shape)
            goff = [0] * t.dim()
            goff[ax] = tp_rank * t.shape[ax]
            gshape[ax] = t.shape[ax] * tp_world
            out[key] = ShardedTensor(key, t, tuple(gshape), tuple(goff), replica_id=dp_rank + extra_replica)
        else:
            out[key] = ShardedTensor(key, t, tuple(t.shape), tuple([0] * t.dim()), replica_id=dp_rank + tp_rank * 1000 + extra_replica)
    return out


def _stacked_layer_key(name: str, layer_numbers: Dict[int, int]):
    """``decoder.layers.3.mlp.linear_fc1.weight`` -> (``decoder.layers.mlp.linear_fc1.weight``, global layer index).
    Names outside ``decoder.layers`` come back unchanged with index None."""
    parts = name.split(".")
    if "layers" in parts:
        i = parts.index("layers")
        if i + 1 < len(parts) and parts[i + 1].isdigit() and int(parts[i + 1]) in layer_numbers:
            g = layer_numbers[int(parts[i + 1])] - 1
            return ".".join(parts[:i + 1] + parts[i + 2:]), g
    return name, None


def _stack(st: ShardedTensor, layer: Optional[int], num_layers: int) -> ShardedTensor:
    """Prepend the layer axis: the chunk becomes row ``layer`` of a [num_layers, ...] global tensor."""
    if layer is None:
        return st
    return ShardedTensor(st.key, st.data.unsqueeze(0), (num_layers,) + tuple(st.global_shape), (layer,) + tuple(st.global_offset),
                         st.replica_id)


def _num_layers(inner) -> int:
    cfg = getattr(inner, "config", None)
    n = getattr(cfg, "num_layers", None)
    if n:
        return int(n)
    return max([l.layer_number for l in inner.decoder.layers] + [0]) if hasattr(inner, "decoder") else 0


def model_sharded_state_dict(model, prefix: str = "") -> Dict[str, ShardedTensor]:
    """One entry per parameter / persistent buffer.  Tensor-parallel parameters carry ``tensor_model_parallel`` and
    ``partition_dim`` attributes (set by the parallel layers) which give their split; stacked expert weights are split
    along the expert axis over expert-parallel ranks; everything else is replicated.  Layer indices become global so
    any pipeline layout maps to the same keys.  (Parameters with ``partition_stride`` > 1, the gated FC1, keep their
    per-rank [gate; up] interleave: they reload under the same tensor-parallel size.)"""
    inner = model.module if hasattr(model, "module") and not hasattr(model, "decoder") else model
    layer_numbers = {}
    if hasattr(inner, "decoder"):
        for i, l in enumerate(inner.decoder.layers):
            layer_numbers[i] = l.layer_number
    init = ps.model_parallel_is_initialized()
    tp_rank = ps.get_tensor_model_parallel_rank() if init else 0
    tp = ps.get_tensor_model_parallel_world_size() if init else 1
    dp_rank = ps.get_data_parallel_rank(with_context_parallel=True) if init else 0
    ep_rank = ps.get_expert_model_parallel_rank() if init else 0
    ep = ps.get_expert_model_parallel_world_size() if init else 1
    edp_rank = ps.get_expert_data_parallel_rank() if init else 0
    out: Dict[str, ShardedTensor] = {}
    items = list(inner.named_parameters()) + [(n, b) for n, b in inner.named_buffers() if b is not None and b.numel() > 0]
    total_layers = _num_layers(inner)
    for name, p in items:
        base, layer = _stacked_layer_key(name, layer_numbers)
        key = prefix + base
        t = p.data if isinstance(p, torch.nn.Parameter) else p
        is_expert = not getattr(p, "allreduce", True)
        if is_expert and t.dim() == 3:
            gshape = (t.shape[0] * ep,) + tuple(t.shape[1:])
            goff = (ep_rank * t.shape[0],) + (0,) * (t.dim() - 1)
            st = ShardedTensor(key, t, gshape, goff, replica_id=edp_rank)
        elif getattr(p, "tensor_model_parallel", False) and tp > 1:
            ax = p.partition_dim
            gshape, goff = list(t.shape), [0] * t.dim()
            gshape[ax] = t.shape[ax] * tp
            goff[ax] = tp_rank * t.shape[ax]
            st = ShardedTensor(key, t, tuple(gshape), tuple(goff), replica_id=dp_rank)
        else:
            st = ShardedTensor(key, t, tuple(t.shape), (0,) * t.dim(), replica_id=dp_rank + 1000 * tp_rank)
        out[key if layer is None else f"{key}@{layer}"] = _stack(st, layer, total_layers)   # dict id; the checkpoint key is st.key
    return out


def optimizer_sharded_state_dict(optimizer, sharding_type: str = "fully_sharded_model_space") -> Dict[str, ShardedTensor]:
    """Optimizer state per parameter as rows of a [tp_world, local_numel] matrix: this rank contributes row ``tp_rank``,
    columns = the part of the flattened parameter its distributed-optimizer shard covers.  Any data-parallel size can
    re-read it; the tensor-parallel size must match (as for ``dp_zero_gather_scatter`` in the reference)."""
    out: Dict[str, ShardedTensor] = {}
    tp_rank = ps.get_tensor_model_parallel_rank()
    tp = ps.get_tensor_model_parallel_world_size()
    for chunk_i, chunk in enumerate(optimizer.model_chunks):
        inner = chunk.module
        layer_numbers = {i: l.layer_number for i, l in enumerate(inner.decoder.layers)} if hasattr(inner, "decoder") else {}
        names = {id(p): _stacked_layer_key(n, layer_numbers) for n, p in inner.named_parameters()}
        total_layers = _num_layers(inner)
        for st in optimizer._all_states():
            if st.buf not in chunk.buffers + chunk.expert_buffers:
                continue
            for p in st.bucket.params:
                ps_, pe_ = st.bucket.param_ranges[id(p)]
                lo, hi = max(ps_, st.lo), min(pe_, st.hi)
                if lo >= hi:
                    continue
                n, layer = names[id(p)]
                split = getattr(p, "tensor_model_parallel", False)
                rows, row = (tp, tp_rank) if split else (1, 0)
                sl = slice(lo - st.lo, hi - st.lo)
                replica = 0 if (split or tp_rank == 0) else tp_rank
                replica += 0 if optimizer.sharded else st.buf.dp_rank
                for kind, src in (("exp_avg", st.m), ("exp_avg_sq", st.v), ("fp32_param", st.master if (st.param16 is not None and st.master is not None) else None),
                                  ("residual", getattr(st, "residual", None)),
                                  ("ema", st.ema)):
                    if src is None:
                        continue
                    key = f"optimizer.state.{kind}.{n}"
                    out[key if layer is None else f"{key}@{layer}"] = _stack(ShardedTensor(key, src[sl].view(1, -1), (rows, pe_ - ps_), (row, lo - ps_), replica_id=replica),
                                      layer, total_layers)
    return out
