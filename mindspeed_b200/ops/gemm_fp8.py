"""Block-scaled fp8 GEMM / grouped GEMM (host side of csrc/kernels/gemm_fp8_sm100.cu) and the fp8 linear autograd.

  fp8_gemm(xq, xs, wq, ws)                  y[M,N] = blockscaled(xq[M,K], wq[N,K]); xs [M,K/128]; ws [N/128,K/128] or,
                                            with ``w_rowwise``, [N,K/128]
  fp8_grouped_gemm(xq, xs, wq, ws, counts)  expert-sorted rows; experts padded to 128-row tiles internally
  Fp8BlockwiseLinearFn                      y = x W^T with all three GEMMs in fp8:
        fprop   x  -> 1x128 along K ; W   -> 128x128            (K-major both)
        dgrad   dy -> 1x128 along N ; W^T -> 128x128            (the transposed weight is quantised separately)
        wgrad   dy^T, x^T -> 1x128 along the token dimension, both row-wise scaled, fp32 accumulation
  On CPU (or for shapes the kernel does not take) the fp32 reference of the same math is used, so the numerics of
  the recipe - not only its speed - are testable without a GPU.
reference: mindspeed/te/pytorch/fp8/recipes/float8_block_scaling_recipe.py:15-26, mindspeed/ops/gmm_mxfp8.py:99-152.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import gemm as G
from . import loader
from .quant import quant_128x128, quant_1x128

_FMT = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def _ref(xq, xs, wq, ws, w_rowwise, out_dtype):
    M, K = xq.shape
    N = wq.shape[0]
    x = (xq.float().view(M, K // 128, 128) * xs.unsqueeze(-1)).view(M, K)
    if w_rowwise:
        w = (wq.float().view(N, K // 128, 128) * ws.unsqueeze(-1)).view(N, K)
    else:
        w = (wq.float().view(N // 128, 128, K // 128, 128) * ws[:, None, :, None]).view(N, K)
    return (x @ w.t()).to(out_dtype)


def _kernel_ok(xq, wq, N, K):
    return xq.is_cuda and loader.lib() is not None and K % 128 == 0 and xq.is_contiguous() and wq.is_contiguous() \
        and xq.dtype in _FMT and wq.dtype in _FMT


def fp8_gemm(xq, xs, wq, ws, out_dtype=torch.bfloat16, w_rowwise: bool = False, out: Optional[torch.Tensor] = None,
             accumulate: bool = False):
    """``out`` (fp32) with ``accumulate`` adds into it (main-grad fusion of the weight gradient)."""
    M, K = xq.shape
    N = wq.shape[0]
    if not _kernel_ok(xq, wq, N, K) or (not w_rowwise and N % 128 != 0):
        y = _ref(xq, xs, wq, ws, w_rowwise, torch.float32)
        if out is not None:
            out.add_(y) if accumulate else out.copy_(y)
            return out
        return y.to(out_dtype)
    L = loader.require_lib()
    xs_t = xs.t().contiguous().float()
    ws_k = ws.t().contiguous().float() if w_rowwise else ws.contiguous().float()
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=xq.device)
    epi = 0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("fp8_gemm writes bf16 or fp32")
    st = G.status_word(xq.device)
    loader.check(L.msb_gemm_fp8_blockscaled(loader.p(xq), loader.p(xs_t), loader.p(wq), loader.p(ws_k), loader.p(out), None,
                                            M, N, K, 1, int(w_rowwise), _FMT[xq.dtype], _FMT[wq.dtype], epi,
                                            ctypes.c_longlong(out.stride(0)), loader.p(st), ctypes.c_void_p(loader.stream_ptr())),
                 "gemm_fp8_blockscaled")
    return out


def fp8_grouped_gemm(xq, xs, wq, ws, tokens_per_expert: Sequence[int], out_dtype=torch.bfloat16):
    """xq [R, K] rows sorted by expert, xs [R, K/128]; wq [G, N, K], ws [G, N/128, K/128] -> [R, N]."""
    counts = [int(c) for c in (tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else tokens_per_expert)]
    Gn, N, K = wq.shape
    R = xq.shape[0]
    if not _kernel_ok(xq, wq, N, K) or N % 128 != 0:
        outs, s = [], 0
        for g, c in enumerate(counts):
            outs.append(_ref(xq[s:s + c], xs[s:s + c], wq[g], ws[g], False, out_dtype))
            s += c
        return torch.cat(outs) if outs else xq.new_zeros(0, N, dtype=out_dtype)
    L = loader.require_lib()
    padded = [((c + 127) // 128) * 128 for c in counts]
    Rp = sum(padded)
    dev = xq.device
    # scatter rows into the padded layout (padding rows are zero with zero scale)
    src_idx, dst_idx, tile_group, s, d = [], [], [], 0, 0
    for g, (c, pc) in enumerate(zip(counts, padded)):
        if c:
            src_idx.append(torch.arange(s, s + c))
            dst_idx.append(torch.arange(d, d + c))
        tile_group += [g] * (pc // 128)
        s += c
        d += pc
    if Rp == 0:
        return xq.new_zeros(0, N, dtype=out_dtype)
    dst = torch.cat(dst_idx).to(dev)
    xq_p = torch.zeros(Rp, K, dtype=torch.uint8, device=dev)
    xq_p[dst] = xq.view(torch.uint8)
    xs_p = torch.zeros(Rp, K // 128, dtype=torch.float32, device=dev)
    xs_p[dst] = xs.float()
    tg = torch.tensor(tile_group, dtype=torch.int32, device=dev)
    out_p = torch.empty(Rp, N, dtype=out_dtype, device=dev)
    st = G.status_word(dev)
    loader.check(L.msb_gemm_fp8_blockscaled(loader.p(xq_p), loader.p(xs_p.t().contiguous()), loader.p(wq.contiguous()),
                                            loader.p(ws.contiguous().float().view(Gn * (N // 128), K // 128)), loader.p(out_p),
                                            loader.p(tg), Rp, N, K, Gn, 0, _FMT[xq.dtype], _FMT[wq.dtype], 0,
                                            ctypes.c_longlong(N), loader.p(st), ctypes.c_void_p(loader.stream_ptr())),
                 "gemm_fp8_blockscaled(grouped)")
    return out_p[dst]


class Fp8BlockwiseLinearFn(torch.autograd.Function):
    """y = x @ w.T with block-scaled fp8 operands in fprop, dgrad and wgrad.  ``wcache`` (dict) keeps the quantised
    weight and its transpose across micro-batches; the owner clears it when the weight changes."""

    @staticmethod
    def forward(ctx, x, w, wcache, grad_dtype):
        x2 = x.reshape(-1, x.shape[-1])
        if wcache is None or "wq" not in wcache:
            wq, ws = quant_128x128(w.detach())
            wtq, wts = quant_128x128(w.detach().t().contiguous())
            if wcache is not None:
                wcache.update(wq=wq, ws=ws, wtq=wtq, wts=wts)
        else:
            wq, ws, wtq, wts = wcache["wq"], wcache["ws"], wcache["wtq"], wcache["wts"]
        xq, xs = quant_1x128(x2)
        y = fp8_gemm(xq, xs, wq, ws, out_dtype=x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)
        ctx.save_for_backward(x2, wtq, wts)
        ctx.x_shape, ctx.w_shape, ctx.grad_dtype, ctx.w_dtype = x.shape, w.shape, grad_dtype, w.dtype
        return y.view(*x.shape[:-1], w.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, wtq, wts = ctx.saved_tensors
        N, K = ctx.w_shape
        dy2 = dy.reshape(-1, N).contiguous()
        M = dy2.shape[0]
        gdt = ctx.grad_dtype or torch.float8_e4m3fn
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, dys = quant_1x128(dy2, dtype=gdt)
            dx = fp8_gemm(dyq, dys, wtq, wts, out_dtype=torch.float32 if dy.dtype == torch.float32 else torch.bfloat16)
            dx = dx.view(ctx.x_shape).to(dy.dtype)
        if ctx.needs_input_grad[1]:
            pad = (-M) % 128
            dyt = torch.nn.functional.pad(dy2, (0, 0, 0, pad)).t().contiguous()      # [N, Mp]
            xt = torch.nn.functional.pad(x2, (0, 0, 0, pad)).t().contiguous()        # [K, Mp]
            dytq, dyts = quant_1x128(dyt, dtype=gdt)
            xtq, xts = quant_1x128(xt)
            dw = fp8_gemm(dytq, dyts, xtq, xts, out_dtype=torch.float32, w_rowwise=True).to(ctx.w_dtype)
        return dx, dw, None, None


def fp8_blockwise_linear(x, w, wcache: Optional[dict] = None, grad_dtype=None):
    if x.shape[-1] % 128 != 0 or w.shape[0] % 128 != 0:
        raise ValueError("the blockwise fp8 recipe needs in/out features that are multiples of 128")
    return Fp8BlockwiseLinearFn.apply(x, w, wcache, grad_dtype)
