"""bf16 GEMM on the hand-written tcgen05 kernel (csrc/kernels/gemm_sm100.cu).

Three entry points cover a linear layer without any transpose copy:
  linear_fwd(x, w)              y  = x @ w.T          x [M,K],  w [N,K]
  linear_dgrad(dy, w)           dx = dy @ w           dy [M,N], w [N,K]
  linear_wgrad(dy, x, acc)      dW = dy.T @ x         dy [M,N], x [M,K]; ``acc`` fp32 [N,K] is accumulated in place
"""
from __future__ import annotations

import ctypes

import torch

from . import loader

EPI_BF16, EPI_F32, EPI_F32_ACC = 0, 1, 2
_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device error word written by a kernel whose bounded wait expired (0 = healthy)."""
    t = _status.get(device)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def check_status(device=None):
    """Synchronising check; raises if any GEMM-class kernel recorded a time-out since the last check."""
    for dev, t in _status.items():
        if device is not None and dev != device:
            continue
        v = int(t[0].item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"sm_100a kernel reported a bounded-wait time-out, code 0x{v:x} on {dev}")


class cta_limit:
    """``with cta_limit(n):`` GEMM-class kernels launched inside use at most ``n`` CTAs (= SMs).  Lets two persistent
    kernels on different streams split the GPU between them."""

    def __init__(self, n: int):
        self.n = int(n)

    def __enter__(self):
        L = loader.require_lib()
        self.prev = L.msb_gemm_get_cta_limit()
        L.msb_gemm_set_cta_limit(self.n)
        return self

    def __exit__(self, *exc):
        loader.require_lib().msb_gemm_set_cta_limit(self.prev)
        return False


class variant:
    """``with variant(v):`` force the plain GEMM onto one kernel: 1 = one-CTA kernel, 2 / 3 = CTA-pair kernel with
    256 x 256 / 256 x 128 tiles, 0 = chosen per shape by the library's time model (the default).  For benchmarks and tests."""

    def __init__(self, v: int):
        self.v = int(v)

    def __enter__(self):
        L = loader.require_lib()
        self.prev = L.msb_gemm_get_variant()
        L.msb_gemm_set_variant(self.v)
        return self

    def __exit__(self, *exc):
        loader.require_lib().msb_gemm_set_variant(self.prev)
        return False


def set_stream_k(on: bool) -> None:
    """Allow (default) or forbid k-block balancing in the accumulate-into-fp32 weight-gradient GEMM.  Forbidding it
    makes the accumulation order, hence the result bits, the same on every run."""
    loader.require_lib().msb_gemm_set_stream_k(1 if on else 0)


def supported(*tensors) -> bool:
    if loader.lib() is None:
        return False
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.data_ptr() % 16 != 0:
            return False
    return True


def _gemm(a, b, d, M, N, K, lda, ldb, ldd, a_mn, b_mn, epi, bias=None):
    L = loader.require_lib()
    st = status_word(a.device)
    ll = ctypes.c_longlong
    loader.check(L.msb_gemm_bf16(loader.p(a), loader.p(b), loader.p(d), loader.p(bias), M, N, K, ll(lda), ll(ldb), ll(ldd),
                                 int(a_mn), int(b_mn), int(epi), loader.p(st), ctypes.c_void_p(loader.stream_ptr())),
                 "gemm_bf16")
    return d


def _2d(t):
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.is_contiguous() else t2.contiguous()


def linear_fwd(x, w, bias=None, out=None):
    x2 = _2d(x)
    M, K = x2.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)  # final shape: never hand back a view
    _gemm(x2, w, out, M, N, K, K, K, N, 0, 0, EPI_BF16, bias)
    return out


def linear_dgrad(dy, w, out=None):
    dy2 = _2d(dy)
    M, N = dy2.shape
    Kout = w.shape[1]
    if out is None:
        out = torch.empty(*dy.shape[:-1], Kout, dtype=torch.bfloat16, device=dy.device)
    # reduction over N: A = dy [M, N] K-major; B = w stored [N(red), Kout] -> MN-major
    _gemm(dy2, w, out, M, Kout, N, N, Kout, Kout, 0, 1, EPI_BF16)
    return out


def linear_wgrad(dy, x, acc=None):
    dy2, x2 = _2d(dy), _2d(x)
    T, N = dy2.shape
    K = x2.shape[1]
    # dW[N, K] = sum_t dy[t, N] x[t, K]: A = dy stored [T(red), N] MN-major; B = x stored [T(red), K] MN-major
    if acc is not None:
        assert acc.dtype == torch.float32 and acc.is_contiguous()
        _gemm(dy2, x2, acc, N, K, T, N, K, K, 1, 1, EPI_F32_ACC)
        return None
    out = torch.empty(N, K, dtype=torch.bfloat16, device=dy.device)
    _gemm(dy2, x2, out, N, K, T, N, K, K, 1, 1, EPI_BF16)
    return out


def shapes_ok(M, N, K) -> bool:
    return M > 0 and N % 8 == 0 and K % 8 == 0 and M % 8 == 0
