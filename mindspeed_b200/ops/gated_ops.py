"""Gated RMSNorm, Sinkhorn normalisation and manifold hyper-connection mixing.

  rms_norm_gated(x, gate, weight, eps)       rmsnorm(x) * weight * silu(gate)    (CUDA: csrc/kernels/gated_ops.cu)
  sinkhorn(logits, iters, eps)               alternating row / column normalisation of exp(logits), n x n with n <= 8
  HyperConnection                            residual mixing across ``hc_mult`` parallel residual streams with a doubly
                                             stochastic (Sinkhorn-projected) stream-mixing matrix per token
reference: mindspeed/lite/ops/triton/fused_norm_gate.py:31-325 (gated norm), mindspeed/lite/ops/triton/sinkhorn.py:11-363 and
mindspeed/lite/ops/triton/mhc/* (pre_bmm / post_bmm1 / post_bmm2 / add: the hyper-connection products).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn as nn

from . import loader
from ._dtypes import code


def rms_norm_gated_ref(x, gate, weight, eps=1e-6):
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * r * weight.float() * torch.nn.functional.silu(gate.float())).to(x.dtype)


class _GatedNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        L = loader.require_lib()
        xc, gc = x.contiguous(), gate.contiguous()
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = weight.to(x.dtype).contiguous()
        loader.check(L.msb_rmsnorm_gated_fwd(loader.p(xc), loader.p(gc), loader.p(w), loader.p(y), loader.p(rstd),
                                             ctypes.c_longlong(rows), cols, ctypes.c_float(eps), code(x.dtype),
                                             ctypes.c_void_p(loader.stream_ptr())), "rmsnorm_gated_fwd")
        ctx.save_for_backward(xc, gc, w, rstd)
        ctx.w_dtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        L = loader.require_lib()
        x, g, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        cols = x.shape[-1]
        rows = x.numel() // cols
        dx, dg = torch.empty_like(x), torch.empty_like(g)
        n_cta = L.msb_rmsnorm_gated_bwd_ctas(ctypes.c_longlong(rows))
        part = torch.empty(n_cta, cols, dtype=torch.float32, device=x.device)
        loader.check(L.msb_rmsnorm_gated_bwd(loader.p(dy), loader.p(x), loader.p(g), loader.p(w), loader.p(rstd), loader.p(dx),
                                             loader.p(dg), loader.p(part), ctypes.c_longlong(rows), cols, code(x.dtype),
                                             ctypes.c_void_p(loader.stream_ptr())), "rmsnorm_gated_bwd")
        return dx, dg, part.sum(0).to(ctx.w_dtype), None


def rms_norm_gated(x, gate, weight, eps: float = 1e-6):
    if loader.use_kernels(x) and x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] <= 12288:
        return _GatedNormFn.apply(x, gate, weight, eps)
    return rms_norm_gated_ref(x, gate, weight, eps)


def sinkhorn_ref(logits, iters: int = 20, eps: float = 1e-6):
    m = torch.exp(logits.float() - logits.float().amax(dim=(-2, -1), keepdim=True))
    for _ in range(iters):
        m = m / (m.sum(-1, keepdim=True) + eps)
        m = m / (m.sum(-2, keepdim=True) + eps)
    return m


class _SinkhornFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, iters, eps):
        L = loader.require_lib()
        lg = logits.float().contiguous()
        n = lg.shape[-1]
        count = lg.numel() // (n * n)
        out = torch.empty_like(lg)
        loader.check(L.msb_sinkhorn_fwd(loader.p(lg), loader.p(out), ctypes.c_longlong(count), n, iters, ctypes.c_float(eps),
                                        ctypes.c_void_p(loader.stream_ptr())), "sinkhorn_fwd")
        ctx.save_for_backward(lg)
        ctx.iters, ctx.eps, ctx.in_dtype = iters, eps, logits.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        L = loader.require_lib()
        (lg,) = ctx.saved_tensors
        n = lg.shape[-1]
        count = lg.numel() // (n * n)
        d = torch.empty_like(lg)
        loader.check(L.msb_sinkhorn_bwd(loader.p(lg), loader.p(dout.float().contiguous()), loader.p(d), ctypes.c_longlong(count), n,
                                        ctx.iters, ctypes.c_float(ctx.eps), ctypes.c_void_p(loader.stream_ptr())), "sinkhorn_bwd")
        return d.to(ctx.in_dtype), None, None


def sinkhorn(logits, iters: int = 20, eps: float = 1e-6):
    """logits [..., n, n] -> approximately doubly stochastic fp32 matrices."""
    if logits.shape[-1] != logits.shape[-2]:
        raise ValueError("sinkhorn expects square matrices")
    if loader.use_kernels(logits) and logits.shape[-1] <= 8 and iters <= 32:
        return _SinkhornFn.apply(logits, iters, eps)
    return sinkhorn_ref(logits, iters, eps)


class HyperConnection(nn.Module):
    """Manifold hyper-connections around a sub-layer ``f``: the residual is kept as ``n`` parallel streams
    H [.., n, h].  Per token, from the (normalised) mean stream:
        a = softmax-free mixing vector  [n]      -> layer input   x = sum_i a_i H_i            ("pre" product)
        B = sinkhorn(W_mix(x~)) [n, n]           -> stream mixing H' = B H                      ("post" product 1)
        c = write vector [n]                     -> H'' = H' + c (outer) f(x)                   ("post" product 2 + add)
    B doubly stochastic keeps the total residual mass constant, which is what makes deep stacks trainable."""

    def __init__(self, hidden_size: int, n_streams: int = 4, sinkhorn_iters: int = 20):
        super().__init__()
        self.n, self.iters = n_streams, sinkhorn_iters
        self.norm_w = nn.Parameter(torch.ones(hidden_size))
        self.read = nn.Linear(hidden_size, n_streams, bias=True)
        self.mix = nn.Linear(hidden_size, n_streams * n_streams, bias=True)
        self.write = nn.Linear(hidden_size, n_streams, bias=True)
        with torch.no_grad():
            for lin in (self.read, self.mix, self.write):
                lin.weight.zero_()
            self.read.bias.fill_(1.0 / n_streams)
            self.write.bias.fill_(1.0)
            self.mix.bias.copy_((torch.eye(n_streams) * 4.0).reshape(-1))      # starts close to the identity mixing

    def forward(self, streams: torch.Tensor, fn):
        """streams [..., n, h] -> same shape; ``fn`` maps [..., h] -> [..., h]."""
        mean = streams.mean(dim=-2)
        xt = mean * torch.rsqrt(mean.float().pow(2).mean(-1, keepdim=True) + 1e-6).to(mean.dtype) * self.norm_w
        a = self.read(xt)                                                     # [..., n]
        x = torch.einsum("...n,...nh->...h", a, streams)
        B = sinkhorn(self.mix(xt).reshape(*xt.shape[:-1], self.n, self.n), self.iters).to(streams.dtype)
        mixed = torch.einsum("...ij,...jh->...ih", B, streams)
        y = fn(x)
        c = self.write(xt)
        return mixed + c.unsqueeze(-1) * y.unsqueeze(-2)

    @staticmethod
    def expand(x: torch.Tensor, n: int) -> torch.Tensor:
        return x.unsqueeze(-2).expand(*x.shape[:-1], n, x.shape[-1]).contiguous()

    @staticmethod
    def collapse(streams: torch.Tensor) -> torch.Tensor:
        return streams.sum(dim=-2)
