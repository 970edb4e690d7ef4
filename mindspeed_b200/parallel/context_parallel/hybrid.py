"""Hybrid (USP) context parallelism: cp = ulysses_degree x ring_degree.  Ulysses groups are contiguous ranks, ring
groups are strided (reference: mindspeed/core/context_parallel/model_parallel_utils.py:59-118,
dot_product_attention.py:210-271)."""
from __future__ import annotations

from .. import parallel_state as ps
from .ring import ring_attention
from .ulysses import ulysses_attention


def hybrid_attention(q, k, v, config, causal=True, softmax_scale=None, layer_number=1):
    ug = ps.get_context_parallel_group_for_hybrid_ulysses()
    rg = ps.get_context_parallel_group_for_hybrid_ring()
    rr = ps.get_context_parallel_for_hybrid_ring_global_ranks()
    ro = ps.get_context_parallel_group_for_hybrid_ring_overlap()

    def inner(qh, kh, vh):
        return ring_attention(qh, kh, vh, config, causal, softmax_scale, layer_number, group=rg, ranks=rr, group_overlap=ro)

    return ulysses_attention(q, k, v, config, ug, causal, softmax_scale, layer_number, inner=inner)
