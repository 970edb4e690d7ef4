"""ctypes loader for the in-tree kernel library."""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "csrc", "libmsb200_kernels.so")
_lock = threading.Lock()
_lib = None
_tried = False


def have_lib() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    """The loaded kernel library, or None when it cannot be used (no GPU)."""
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    with _lock:
        if _lib is not None or _tried:
            return _lib
        _tried = True
        if not torch.cuda.is_available():
            return None
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing on a machine with a GPU; build it with "
                "`python -m mindspeed_b200.ops.build` (or __graft_entry__.build())")
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        _lib.msb_launch_count.restype = ctypes.c_ulonglong
        _lib.msb_last_error.restype = ctypes.c_char_p
    return _lib


def require_lib():
    l = lib()
    if l is None:
        raise RuntimeError("the sm_100a kernel library needs a CUDA device")
    return l


def use_kernels(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a GPU (then the kernel library must be present)."""
    return t.is_cuda and lib() is not None


def launch_count() -> int:
    l = lib()
    return int(l.msb_launch_count()) if l is not None else 0


def reset_launch_count() -> None:
    l = lib()
    if l is not None:
        l.msb_reset_launch_count()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str):
    if rc != 0:
        l = lib()
        msg = l.msb_last_error().decode() if l is not None else ""
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def p(t):
    """Raw device pointer as ctypes void*."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())
