"""Adam with quantised moments: exp_avg / exp_avg_sq are stored as fp8 (e4m3 for m, e5m2-range-safe e4m3 with sqrt
companding for v) with one fp32 scale per block of 128 elements (``fp8``) or 32 elements with power-of-two scales
(``mxfp8``).  Each step dequantises a slice, runs the fused fp32 AdamW kernel and requantises; state memory drops from
8 to ~2.06 bytes per parameter (reference: mindspeed/core/optimizer/low_precision/quant_adamw.py:14-526, ScaleMeta).
"""
from __future__ import annotations

import torch

from ..ops import adam as adam_ops
from ..ops.quant import dequantize_blockwise, quantize_blockwise
from .distrib_optimizer import DistributedOptimizer


class _QState:
    def __init__(self, n, dev, block, pow2, signed_sqrt):
        self.n, self.block, self.pow2, self.sqrt = n, block, pow2, signed_sqrt
        self.q, self.scale = quantize_blockwise(torch.zeros(n, device=dev), block, pow2)

    def load(self, sl):
        x = dequantize_blockwise(self.q, self.scale, self.block)[sl]
        return x * x if self.sqrt else x

    def store(self, full):
        x = full.clamp_min(0).sqrt() if self.sqrt else full
        self.q, self.scale = quantize_blockwise(x, self.block, self.pow2)


class QuantStateDistributedOptimizer(DistributedOptimizer):
    def __init__(self, config, model_chunks, *a, **k):
        super().__init__(config, model_chunks, *a, **k)
        block, pow2 = (32, True) if config.quant_states == "mxfp8" else (128, False)
        for st in self._all_states():
            n = st.m.numel()
            st.qm = _QState(n, st.m.device, block, pow2, signed_sqrt=False)
            st.qv = _QState(n, st.m.device, block, pow2, signed_sqrt=True)   # second moment: store its square root
            st.m = st.v = None

    @torch.no_grad()
    def step(self):
        # materialise the fp32 moments of every bucket, run the standard step on them, requantise: the resident state
        # between steps is the quantised one; during the step the fp32 moments of all buckets exist at once
        for st in self._all_states():
            st.m = st.qm.load(slice(None)).contiguous()
            st.v = st.qv.load(slice(None)).contiguous()
        out = super().step()
        for st in self._all_states():
            st.qm.store(st.m)
            st.qv.store(st.v)
            st.m = st.v = None
        return out
