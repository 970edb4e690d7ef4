""""Virtual" optimizer state: Adam moments placed in host memory that the GPU addresses directly (pinned, mapped),
so no explicit swap is scheduled; each pipeline stage chooses what fraction of its moments goes there
(``--virtual-optimizer f0 f1 ...``).  reference: mindspeed/core/optimizer/virtual_optimizer/virtual_adam.py:10-190,
which uses ``torch_npu.empty_with_swapped_memory``; on CUDA the equivalent is pinned host memory accessed through
unified addressing (reads and writes travel over PCIe / C2C at kernel time)."""
from __future__ import annotations

import torch

from ..parallel import parallel_state as ps
from .distrib_optimizer import DistributedOptimizer


def empty_mapped(n, dtype=torch.float32):
    """Pinned host tensor plus a CUDA tensor aliasing it (zero-copy)."""
    host = torch.zeros(n, dtype=dtype, pin_memory=True)
    if not torch.cuda.is_available():
        return host, host
    from ..parallel.symm_mem import _RawCuda
    dev = torch.as_tensor(_RawCuda(host.data_ptr(), n * host.element_size()), device="cuda").view(dtype)
    return host, dev


class VirtualDistributedOptimizer(DistributedOptimizer):
    def __init__(self, config, model_chunks, fractions, *a, **k):
        super().__init__(config, model_chunks, *a, **k)
        stage = ps.get_pipeline_model_parallel_rank()
        frac = fractions[min(stage, len(fractions) - 1)] if fractions else 0.0
        self._keep = []
        budget = frac * sum(st.m.numel() for st in self._all_states())
        for st in self._all_states():
            if budget <= 0:
                break
            n = st.m.numel()
            for name in ("m", "v"):
                host, dev = empty_mapped(n)
                dev.copy_(getattr(st, name))
                setattr(st, name, dev)
                self._keep.append(host)
            budget -= n
