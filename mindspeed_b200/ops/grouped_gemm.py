"""Grouped GEMM over expert-sorted rows: y[rows_e] = x[rows_e] @ W[e]   (W stacked [E, K, N]).

On a GPU forward, data gradient and weight gradient are each ONE launch of the CTA-pair grouped kernel
(csrc/kernels/gemm2_grouped_sm100.cu) over all experts; the experts' row ranges travel as an int32 prefix-sum tensor on the
device, so a ``tokens_per_expert`` tensor is never read back to the host.  The weight gradient accumulates straight into the
fp32 ``main_grad`` of the stacked weight when present; its reduction runs over the whole 64-row blocks of every expert in
the main launch and over a zero-padded copy of the remaining (< 64) rows per expert in a second, small launch.
The CPU path is the eager loop and serves as the oracle.  reference semantics: npu_gmm / npu_gmm_backward
(mindspeed/ops/gmm.py:20-175, mindspeed/ops/csrc/cann/gmm.cpp:169-300: dx = dy W^T, dw = x^T dy grouped on K).
"""
from __future__ import annotations

import ctypes

import torch

from . import gemm as G
from . import loader

TAIL = 64      # reduction block of the weight-gradient kernel


def _sizes(tokens_per_expert):
    return tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else list(tokens_per_expert)


def _offsets(tokens_per_expert, device):
    """int32 [E + 1] prefix sums on ``device`` without a host round trip when the counts already live there."""
    if torch.is_tensor(tokens_per_expert):
        t = tokens_per_expert.to(device=device, dtype=torch.int32)
    else:
        t = torch.tensor(list(tokens_per_expert), dtype=torch.int32, device=device)
    offs = torch.zeros(t.numel() + 1, dtype=torch.int32, device=device)
    torch.cumsum(t, 0, out=offs[1:])
    return offs


def _use_kernel(x, w):
    return (x.is_cuda and loader.lib() is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _rows(x, w, y, offs, n_out, k_red, w_is_kn):
    L = loader.require_lib()
    st = G.status_word(x.device)
    loader.check(L.msb_grouped_gemm_rows(loader.p(x), loader.p(w), loader.p(y), loader.p(offs), w.shape[0], x.shape[0], n_out, k_red,
                                         int(w_is_kn), loader.p(st), ctypes.c_void_p(loader.stream_ptr())), "grouped_gemm_rows")
    return y


def _wgrad(x, dy, dw, offs, epilogue):
    L = loader.require_lib()
    st = G.status_word(x.device)
    loader.check(L.msb_grouped_gemm_wgrad(loader.p(x), loader.p(dy), loader.p(dw), loader.p(offs), dw.shape[0], x.shape[0], x.shape[1],
                                          dy.shape[1], int(epilogue), loader.p(st), ctypes.c_void_p(loader.stream_ptr())),
                 "grouped_gemm_wgrad")


def grouped_wgrad_acc(x, dy, offs, acc):
    """acc[e] (fp32 [E, K, N]) += x[rows of e]^T @ dy[rows of e], rows given by the device prefix sums ``offs``."""
    E = acc.shape[0]
    _wgrad(x, dy, acc, offs, G.EPI_F32_ACC)                  # whole 64-row blocks of every expert
    # the < 64 trailing rows of every expert, gathered into zero-padded [E, 64, .] copies (all on the device)
    end = offs[1:].long()
    n = end - offs[:-1].long()
    tail = n % TAIL
    r = torch.arange(TAIL, device=x.device).view(1, TAIL)
    idx = (end - tail).view(E, 1) + r
    valid = r < tail.view(E, 1)
    idx = torch.where(valid, idx, torch.zeros_like(idx)).view(-1)
    xt = x.index_select(0, idx) * valid.view(-1, 1).to(x.dtype)
    dyt = dy.index_select(0, idx)
    offs2 = torch.arange(E + 1, device=x.device, dtype=torch.int32) * TAIL
    _wgrad(xt, dyt, acc, offs2, G.EPI_F32_ACC)


def grouped_gemm_ref(x, w, tokens_per_expert):
    outs, start = [], 0
    for e, n in enumerate(_sizes(tokens_per_expert)):
        outs.append(x[start:start + n] @ w[e])
        start += n
    return torch.cat(outs, dim=0) if outs else x.new_zeros(0, w.shape[2])


class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offs):
        ctx.save_for_backward(x, w, offs)
        K, N = w.shape[1], w.shape[2]
        out = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        # y = x_e [n, K] @ W_e [K, N]: W stored [K(red), N]
        return _rows(x, w, out, offs, N, K, True)

    @staticmethod
    def backward(ctx, dy):
        x, w, offs = ctx.saved_tensors
        dy = dy.contiguous()
        K, N = w.shape[1], w.shape[2]
        dx = torch.empty_like(x)
        # dx_e [n, K] = dy_e [n, N] @ W_e^T: W_e stored [K(out), N(red)]
        _rows(dy, w, dx, offs, K, N, False)
        main_grad = getattr(w, "main_grad", None)
        fuse = main_grad is not None and main_grad.dtype == torch.float32 and main_grad.is_contiguous()
        if fuse:
            grouped_wgrad_acc(x, dy, offs, main_grad)
            w.grad_added_to_main_grad = True
            cb = getattr(w, "_main_grad_ready_cb", None)
            if cb is not None:
                cb(w)
            return dx, None, None
        acc = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        grouped_wgrad_acc(x, dy, offs, acc)
        return dx, acc.to(w.dtype), None


def grouped_gemm(x, w, tokens_per_expert, trans_b=False):
    """``tokens_per_expert``: list or tensor [E]; rows of ``x`` beyond their sum are left alone (their outputs are
    unspecified), which lets callers pass a fixed-capacity buffer."""
    if trans_b:
        w = w.transpose(1, 2)
    if _use_kernel(x, w) and w.is_contiguous() and x.is_contiguous() and x.shape[0] > 0:
        return _GroupedGemm.apply(x, w, _offsets(tokens_per_expert, x.device))
    return grouped_gemm_ref(x, w, _sizes(tokens_per_expert))
