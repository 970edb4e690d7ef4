"""Muon: momentum followed by Newton-Schulz orthogonalisation of each 2-D weight update.

  m <- mu * m + g ;  u = nesterov ? g + mu * m : m ;  U = NS_k(u) ;  W <- W * (1 - lr*wd) - lr * scale(U)
Newton-Schulz iterates X <- a X + (b A + c A^2) X with A = X X^T on the spectrally normalised update; coefficient
sets "simple" (cubic), "quintic" (Keller Jordan) and "polar_express" are available.  Tensor-parallel weights:
  blockwise    each rank orthogonalises its own shard (no communication)
  duplicated   all-gather the shards, orthogonalise the full matrix everywhere, keep the local slice
  distributed  Gram matrices X X^T are all-reduced so the iteration acts on the full matrix while X stays sharded
1-D parameters, embeddings and the output layer use AdamW (``--muon-scalar-optimizer``).  QKV weights are split into
their q / k / v blocks first unless ``--muon-no-split-qkv``.
reference: mindspeed/core/optimizer/muon/muon_utils.py:67-211, emerging_optimizers.py:125-284,
orthogonalized_optimizer.py:39-249.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

_COEFFS = {
    "simple": [(1.5, -0.5, 0.0)],
    "quintic": [(3.4445, -4.7750, 2.0315)],
    "polar_express": [(8.2051, -22.9019, 16.4607), (4.0664, -2.8612, 0.5184), (3.9096, -2.8234, 0.5250),
                      (3.2856, -2.4153, 0.4853), (2.2779, -1.6198, 0.3985), (1.8726, -1.2307, 0.3585),
                      (1.8564, -1.2132, 0.3568), (1.8750, -1.2500, 0.3750)],
}


def newton_schulz(x: torch.Tensor, steps: int = 5, coefficient_type: str = "quintic", tp_group=None, partition_dim: Optional[int] = None,
                  eps: float = 1e-7) -> torch.Tensor:
    """Approximate the orthogonal polar factor of ``x`` [rows, cols].  With ``tp_group`` the matrix is sharded along
    ``partition_dim`` and the Gram matrices / norm are all-reduced (the "distributed" mode)."""
    dtype = x.dtype
    X = x.float()
    transposed = False
    # work on the wide orientation so that A = X X^T is the small Gram matrix
    rows, cols = X.shape
    full_rows = rows * (dist.get_world_size(tp_group) if (tp_group is not None and partition_dim == 0) else 1)
    full_cols = cols * (dist.get_world_size(tp_group) if (tp_group is not None and partition_dim == 1) else 1)
    if full_rows > full_cols:
        X, transposed = X.t(), True
        if partition_dim is not None:
            partition_dim = 1 - partition_dim
    nrm2 = X.pow(2).sum()
    if tp_group is not None:
        dist.all_reduce(nrm2, group=tp_group)
    X = X / (nrm2.sqrt() + eps)
    coeffs = _COEFFS[coefficient_type]
    for i in range(steps):
        a, b, c = coeffs[min(i, len(coeffs) - 1)]
        if tp_group is not None and partition_dim == 1:
            A = X @ X.t()                      # partial Gram over the sharded columns
            dist.all_reduce(A, group=tp_group)
            B = b * A + c * (A @ A)
            X = a * X + B @ X
        elif tp_group is not None and partition_dim == 0:
            # rows sharded: gather the small side instead (X^T X is [cols, cols], all ranks share it)
            G = X.t() @ X
            dist.all_reduce(G, group=tp_group)
            B = b * G + c * (G @ G)
            X = a * X + X @ B
        else:
            A = X @ X.t()
            B = b * A + c * (A @ A)
            X = a * X + B @ X
    if transposed:
        X = X.t()
    return X.to(dtype)


def muon_scale(shape, mode: str = "spectral", extra: float = 1.0) -> float:
    r, c = shape
    if mode == "spectral":
        return extra * max(1.0, r / c) ** 0.5
    if mode == "unit_rms_norm":
        return extra * (r / c) ** 0.5
    if mode == "shape_scaling":
        return extra * max(r, c) ** 0.5
    raise ValueError(mode)


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr=2e-2, momentum=0.95, nesterov=True, weight_decay=0.0, ns_steps=5, coefficient_type="quintic",
                 scale_mode="spectral", extra_scale_factor=1.0, tp_mode="blockwise", tp_group=None, split_qkv=None):
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay, ns_steps=ns_steps,
                        coefficient_type=coefficient_type, scale_mode=scale_mode, extra_scale_factor=extra_scale_factor)
        super().__init__(params, defaults)
        self.tp_mode, self.tp_group, self.split_qkv = tp_mode, tp_group, split_qkv

    def _orth(self, u, p, group):
        tp = self.tp_group is not None and getattr(p, "tensor_model_parallel", False) and dist.get_world_size(self.tp_group) > 1
        kw = dict(steps=group["ns_steps"], coefficient_type=group["coefficient_type"])
        if not tp or self.tp_mode == "blockwise":
            return newton_schulz(u, **kw)
        dim = p.partition_dim
        if self.tp_mode == "distributed":
            return newton_schulz(u, tp_group=self.tp_group, partition_dim=dim, **kw)
        parts = [torch.empty_like(u) for _ in range(dist.get_world_size(self.tp_group))]
        dist.all_gather(parts, u.contiguous(), group=self.tp_group)
        full = newton_schulz(torch.cat(parts, dim=dim), **kw)
        return full.chunk(len(parts), dim=dim)[dist.get_rank(self.tp_group)].contiguous()

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            for p in group["params"]:
                g = getattr(p, "main_grad", None) if p.grad is None else p.grad
                if g is None:
                    continue
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                buf = st["momentum_buffer"]
                buf.mul_(group["momentum"]).add_(g.float())
                u = g.float() + group["momentum"] * buf if group["nesterov"] else buf
                u2 = u.reshape(u.shape[0], -1)
                blocks = self.split_qkv(p) if (self.split_qkv is not None) else None
                if blocks:
                    outs = [self._orth(u2[a:b], p, group) * muon_scale((b - a, u2.shape[1]), group["scale_mode"], group["extra_scale_factor"])
                            for a, b in blocks]
                    upd = torch.cat(outs, dim=0)
                else:
                    upd = self._orth(u2, p, group) * muon_scale(u2.shape, group["scale_mode"], group["extra_scale_factor"])
                p.mul_(1.0 - group["lr"] * group["weight_decay"])
                p.add_(upd.reshape(p.shape).to(p.dtype), alpha=-group["lr"])
        return None


class SwapMuon(Muon):
    """Muon whose momentum buffers live in pinned host memory: each step copies a parameter's buffer to the device on a
    side stream while the previous parameter is being orthogonalised, and writes it back afterwards, so the device
    only ever holds two momentum buffers (reference: the swap variant of the reference's Muon, --swap-optimizer with
    --optimizer-selection muon)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def _host_buffer(self, p):
        st = self.state[p]
        if "momentum_host" not in st:
            st["momentum_host"] = torch.zeros(p.shape, dtype=torch.float32, device="cpu",
                                              pin_memory=torch.cuda.is_available() and p.is_cuda)
        return st["momentum_host"]

    @torch.no_grad()
    def step(self, closure=None):
        items = [(g, p) for g in self.param_groups for p in g["params"]
                 if (p.grad is not None or getattr(p, "main_grad", None) is not None)]
        if not items:
            return None

        def fetch(p):
            h = self._host_buffer(p)
            if not p.is_cuda:
                return h
            with torch.cuda.stream(self._stream):
                return h.to(p.device, non_blocking=True)

        nxt = fetch(items[0][1])
        for i, (group, p) in enumerate(items):
            if p.is_cuda:
                torch.cuda.current_stream().wait_stream(self._stream)
            buf = nxt
            if i + 1 < len(items):
                nxt = fetch(items[i + 1][1])          # prefetch overlaps this parameter's Newton-Schulz iterations
            g = p.grad if p.grad is not None else p.main_grad
            buf.mul_(group["momentum"]).add_(g.float())
            u = g.float() + group["momentum"] * buf if group["nesterov"] else buf
            u2 = u.reshape(u.shape[0], -1)
            upd = self._orth(u2, p, group) * muon_scale(u2.shape, group["scale_mode"], group["extra_scale_factor"])
            p.mul_(1.0 - group["lr"] * group["weight_decay"])
            p.add_(upd.reshape(p.shape).to(p.dtype), alpha=-group["lr"])
            h = self._host_buffer(p)
            if p.is_cuda:
                self._stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._stream):
                    h.copy_(buf, non_blocking=True)
                buf.record_stream(self._stream)
            elif buf is not h:
                h.copy_(buf)
        return None


class ChainedOptimizer:
    """Several optimizers stepped together (Megatron ``ChainedOptimizer`` surface)."""

    def __init__(self, optimizers: List):
        self.chained = optimizers
        self.param_groups = [g for o in optimizers for g in o.param_groups]
        self.step_count = 0

    def zero_grad(self, set_to_none=True):
        for o in self.chained:
            o.zero_grad(set_to_none)

    def step(self):
        self.step_count += 1
        for o in self.chained:
            o.step()
        return True, None, None

    def state_dict(self):
        return [o.state_dict() for o in self.chained]

    def load_state_dict(self, sd):
        for o, s in zip(self.chained, sd):
            o.load_state_dict(s)


def build_muon_optimizer(config, model_chunks):
    """2-D hidden weights -> Muon; embeddings, output layer, norms and biases -> AdamW.  Gradients are taken from the
    data-parallel buffers' ``main_grad`` (reduced before the step)."""
    from ..parallel import parallel_state as ps
    from .adamw import AdamW
    from ..training.global_vars import get_args
    try:
        a = get_args()
    except RuntimeError:
        a = None
    g = lambda k, d: getattr(a, k, d) if a is not None else d
    muon_p, adam_p = [], []
    for chunk in model_chunks:
        for n, p in chunk.module.named_parameters():
            if p.dim() >= 2 and "embedding" not in n and "output_layer" not in n and "router" not in n:
                muon_p.append(p)
            else:
                adam_p.append(p)
    tp_group = ps.get_tensor_model_parallel_group(check_initialized=False)
    # --muon-fp32-matmul-prec: precision of the fp32 matmuls of the Newton-Schulz iteration (low = tf32 allowed)
    prec = g("muon_fp32_matmul_prec", "medium")
    torch.set_float32_matmul_precision({"low": "medium", "medium": "high", "high": "highest"}.get(prec, "high"))
    if g("muon_scalar_optimizer", "adam") not in ("adam", "adamw"):
        raise NotImplementedError("--muon-scalar-optimizer: only adam is available for the non-matrix parameters")
    split = None
    if g("muon_split_qkv", True):
        def split(p):
            """Row ranges of the q / k / v blocks of a fused QKV weight (None for other parameters)."""
            blocks = getattr(p, "qkv_row_blocks", None)
            return blocks
    muon = Muon(muon_p, lr=config.lr, momentum=g("muon_momentum", 0.95), nesterov=g("muon_nesterov", False),
                weight_decay=config.weight_decay, ns_steps=g("muon_num_ns_steps", 5), coefficient_type=g("muon_coefficient_type", "quintic"),
                scale_mode=g("muon_scale_mode", "spectral"), extra_scale_factor=g("muon_extra_scale_factor", 1.0),
                tp_mode=g("muon_tp_mode", "blockwise"), tp_group=tp_group, split_qkv=split)
    adam = AdamW(adam_p, lr=config.lr, betas=(config.adam_beta1, config.adam_beta2), eps=config.adam_eps, weight_decay=0.0)

    class _MainGradBridge(ChainedOptimizer):
        def step(self):
            for chunk in model_chunks:
                for p in chunk.module.parameters():
                    if hasattr(p, "main_grad"):
                        p.grad = p.main_grad.to(p.dtype)
            out = super().step()
            for chunk in model_chunks:
                for p in chunk.module.parameters():
                    p.grad = None
            return out

        def get_loss_scale(self):
            return torch.ones(1)

        def reload_model_params(self):
            pass

    return _MainGradBridge([muon, adam])
