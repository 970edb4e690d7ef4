"""DeepSpeed-style MoE layer: ``MoE`` -> ``MOELayer`` (dispatch einsum / all-to-all / experts / combine) with a
``TopKGate`` (top-1 / top-2 gating with capacity, random token selection off, load-balancing auxiliary loss).

Dispatch is dense: a [tokens, experts, capacity] one-hot routes tokens into fixed-capacity expert buffers, which is
what makes the all-to-all shapes static (the property the "pipe experts" / "ampipe" variants of the reference rely on
to chunk the exchange).  ``pipe_experts`` splits the capacity dimension into chunks so that chunk i's all-to-all can
overlap chunk i-1's expert compute.
reference: mindspeed/moe/{moe.py,moe_layer.py,gate.py,experts.py,pipe_experts.py,ampipe/*} (960 lines).
"""
from .gate import TopKGate, top1gating, top2gating
from .layer import MoE, MOELayer, Experts

__all__ = ["TopKGate", "top1gating", "top2gating", "MoE", "MOELayer", "Experts"]
