"""FLOP counting for MFU / HFU (reference: mindspeed/functional/tflops_calculate/tflops_utils.py:5-60).

``FlopsCounter`` is started / stopped around a train step; op wrappers call ``add_mm`` / ``add_attention`` / ``add_gmm``.
Inside recompute (``recompute_scope``) FLOPs count towards HFU only."""
from __future__ import annotations

import contextlib

from .host_lib import host_lib


class FlopsCounter:
    def start(self):
        host_lib().msb_flops_start()

    def stop(self):
        host_lib().msb_flops_stop()

    @property
    def model_flops(self):
        return int(host_lib().msb_flops_model())

    @property
    def hardware_flops(self):
        return int(host_lib().msb_flops_hardware())


def add_mm(m, n, k):
    L = host_lib()
    L.msb_flops_add(L.msb_mm_flop(m, n, k))


def add_attention(b, heads, sq, sk, d, dv, causal, backward=False):
    L = host_lib()
    fn = L.msb_flash_attention_backward_flop if backward else L.msb_flash_attention_forward_flop
    L.msb_flops_add(fn(b, heads, sq, sk, d, dv, 0.5 if causal else 1.0))


def add_gmm(group_rows, k, n):
    import ctypes
    L = host_lib()
    arr = (ctypes.c_longlong * len(group_rows))(*[int(x) for x in group_rows])
    L.msb_flops_add(L.msb_gmm_flop(arr, len(group_rows), ctypes.c_longlong(k), ctypes.c_longlong(n)))


@contextlib.contextmanager
def recompute_scope():
    L = host_lib()
    L.msb_flops_enter_recompute()
    try:
        yield
    finally:
        L.msb_flops_exit_recompute()
