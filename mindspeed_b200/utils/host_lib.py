"""ctypes loader of the host-side native library (csrc/host/*.cpp -> libmsb200_host.so)."""
import ctypes
import os

_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "libmsb200_host.so")
_lib = None


def host_lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            from ..ops.build import build
            build()
        _lib = ctypes.CDLL(_PATH)
        for name in ("msb_mm_flop", "msb_bmm_flop", "msb_coc_flop", "msb_flash_attention_forward_flop",
                     "msb_flash_attention_backward_flop", "msb_gmm_flop", "msb_gmm_add_flop", "msb_flops_model", "msb_flops_hardware"):
            getattr(_lib, name).restype = ctypes.c_longlong
        _lib.msb_flash_attention_forward_flop.argtypes = [ctypes.c_longlong] * 6 + [ctypes.c_double]
        _lib.msb_flash_attention_backward_flop.argtypes = [ctypes.c_longlong] * 6 + [ctypes.c_double]
        _lib.msb_mm_flop.argtypes = [ctypes.c_longlong] * 3
        _lib.msb_bmm_flop.argtypes = [ctypes.c_longlong] * 4
        _lib.msb_flops_add.argtypes = [ctypes.c_longlong]
    return _lib
