"""Grouped GEMM over expert-sorted rows: y[rows_e] = x[rows_e] @ W[e]   (W stacked [E, K, N]).

Forward, data gradient and weight gradient each run on the tcgen05 GEMM kernel per expert on a GPU
(the weight gradient accumulates straight into the fp32 ``main_grad`` slice of the expert when present); the CPU
path is the eager loop and serves as the oracle.  reference semantics: npu_gmm / npu_gmm_backward
(mindspeed/ops/gmm.py:20-175, mindspeed/ops/csrc/cann/gmm.cpp:169-300: dx = dy W^T, dw = x^T dy grouped on K).
"""
from __future__ import annotations

import torch

from . import gemm as G
from . import loader


def _sizes(tokens_per_expert):
    return tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)


def _use_kernel(x, w):
    return (x.is_cuda and loader.lib() is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0)


def grouped_gemm_ref(x, w, tokens_per_expert):
    outs, start = [], 0
    for e, n in enumerate(_sizes(tokens_per_expert)):
        outs.append(x[start:start + n] @ w[e])
        start += n
    return torch.cat(outs, dim=0) if outs else x.new_zeros(0, w.shape[2])


class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sizes):
        ctx.sizes = sizes
        ctx.save_for_backward(x, w)
        out = torch.empty(x.shape[0], w.shape[2], dtype=x.dtype, device=x.device)
        start = 0
        for e, n in enumerate(sizes):
            if n > 0:
                # y = x_e [n,K] @ W_e [K,N]: B stored [K(red), N] -> MN-major, same form as a data-gradient GEMM
                G._gemm(x[start:start + n], w[e], out[start:start + n], n, w.shape[2], w.shape[1], w.shape[1], w.shape[2],
                        w.shape[2], 0, 1, G.EPI_BF16)
            start += n
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        main_grad = getattr(w, "main_grad", None)
        fuse = main_grad is not None and main_grad.dtype == torch.float32
        dw = None if fuse else torch.zeros_like(w)
        start = 0
        K, N = w.shape[1], w.shape[2]
        for e, n in enumerate(ctx.sizes):
            if n > 0:
                dye, xe = dy[start:start + n], x[start:start + n]
                # dx_e [n,K] = dy_e [n,N] @ W_e^T: B = W_e stored [K(out), N(red)] -> K-major
                G._gemm(dye, w[e], dx[start:start + n], n, K, N, N, N, K, 0, 0, G.EPI_BF16)
                # dW_e [K,N] = x_e^T [K,n] @ dy_e [n,N]: both operands MN-major (reduction over rows)
                if n % 8 == 0:
                    if fuse:
                        G._gemm(xe, dye, main_grad[e], K, N, n, K, N, N, 1, 1, G.EPI_F32_ACC)
                    else:
                        G._gemm(xe, dye, dw[e], K, N, n, K, N, N, 1, 1, G.EPI_BF16)
                else:
                    t = xe.t().float() @ dye.float()
                    if fuse:
                        main_grad[e].add_(t)
                    else:
                        dw[e].copy_(t)
            start += n
        if fuse:
            w.grad_added_to_main_grad = True
            cb = getattr(w, "_main_grad_ready_cb", None)
            if cb is not None:
                cb(w)
        return dx, dw, None


def grouped_gemm(x, w, tokens_per_expert, trans_b=False):
    if trans_b:
        w = w.transpose(1, 2)
    sizes = _sizes(tokens_per_expert)
    if _use_kernel(x, w) and w.is_contiguous() and x.is_contiguous():
        return _GroupedGemm.apply(x, w, sizes)
    return grouped_gemm_ref(x, w, sizes)
