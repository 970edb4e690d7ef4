"""Context parallelism: ring (double ring), Ulysses, hybrid, KV-allgather, adaptive, Hamilton (multi-cycle ring).

``dispatch_context_parallel_attention`` is the single entry used by the attention module
(reference: mindspeed/core/context_parallel/dot_product_attention.py:134-322).
"""
from __future__ import annotations

from .. import parallel_state as ps


def dispatch_context_parallel_attention(q, k, v, config, causal=True, softmax_scale=None, attention_mask=None,
                                        layer_number=1):
    algo = getattr(config, "context_parallel_algo", "megatron_cp_algo")
    if algo == "megatron_cp_algo":
        from .ring import ring_attention
        return ring_attention(q, k, v, config, causal=causal, softmax_scale=softmax_scale, layer_number=layer_number)
    if algo == "ulysses_cp_algo":
        from .ulysses import ulysses_attention
        return ulysses_attention(q, k, v, config, ps.get_context_parallel_group(), causal=causal,
                                 softmax_scale=softmax_scale, layer_number=layer_number)
    if algo == "hybrid_cp_algo":
        from .hybrid import hybrid_attention
        return hybrid_attention(q, k, v, config, causal=causal, softmax_scale=softmax_scale, layer_number=layer_number)
    if algo == "kvallgather_cp_algo":
        from .kvallgather import kv_allgather_attention
        return kv_allgather_attention(q, k, v, config, softmax_scale=softmax_scale)
    if algo == "hamilton_cp_algo":
        from .hamilton import hamilton_attention
        return hamilton_attention(q, k, v, config, causal=causal, softmax_scale=softmax_scale)
    if algo in ("adaptive_cp_algo", "hybrid_adaptive_cp_algo"):
        from .adaptive import adaptive_attention
        return adaptive_attention(q, k, v, config, attention_mask, softmax_scale=softmax_scale)
    raise ValueError(f"unknown context parallel algorithm {algo}")
