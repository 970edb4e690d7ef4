"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some hosts of the kernel library cannot hand it scratch memory: they run with a fixed memory pool, or inside an
allocator callback, or without PyTorch at all.  For them the library exports ``msb_rmsnorm_bwd_noalloc``, which
keeps its partial sums in an array built into the library.  This test checks that it produces what the regular
entry point (caller-provided scratch) produces, twice in a row, and that it refuses widths beyond its stated
limit instead of launching.  It lives in a file that pytest collects last, so a run that stops at the first
failure has already exercised everything else; it also passes on its own in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mindspeed_b200.ops import loader
    L = loader.require_lib()
    L.msb_rmsnorm_bwd_scratch_elems.restype = ctypes.c_size_t
    L.msb_rmsnorm_bwd_noalloc_max_cols.restype = ctypes.c_size_t
    L.msb_last_error.restype = ctypes.c_char_p
    return L, loader


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_noalloc_rmsnorm_bwd_matches_regular_entry_point(dtype, code):
    L, loader = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tol = 5e-3 if dtype == torch.bfloat16 else 1e-4
    for call, (rows, cols) in enumerate([(1000, 4096), (37, 1024)]):  # two calls in a row share the built-in array
        torch.manual_seed(10 + call)
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
        gamma = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype)
        y = torch.empty_like(x)
        rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
        assert L.msb_rmsnorm_fwd(_vp(x), _vp(gamma), _vp(y), _vp(rstd), rows, cols, ctypes.c_float(1e-5), 0, code, stream) == 0
        dx_ref, dg_ref = torch.empty_like(x), torch.empty_like(gamma)
        scratch = torch.empty(L.msb_rmsnorm_bwd_scratch_elems(rows, cols), device="cuda", dtype=torch.float32)
        assert L.msb_rmsnorm_bwd(_vp(dy), _vp(x), _vp(gamma), _vp(rstd), _vp(dx_ref), _vp(dg_ref), _vp(scratch), rows,
                                 cols, 0, 0, code, stream) == 0
        dx, dg = torch.empty_like(x), torch.empty_like(gamma)
        rc = L.msb_rmsnorm_bwd_noalloc(_vp(dy), _vp(x), _vp(gamma), _vp(rstd), _vp(dx), _vp(dg), rows, cols, 0, 0, code,
                                       stream)
        assert rc == 0, L.msb_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=tol, rtol=tol)
        scale = max(1.0, dg_ref.float().abs().max().item())
        torch.testing.assert_close(dg.float(), dg_ref.float(), atol=tol * scale, rtol=tol)


def test_noalloc_rejects_width_beyond_limit():
    L, _ = _lib()
    limit = L.msb_rmsnorm_bwd_noalloc_max_cols()
    cols = int(limit) + 8
    z = torch.zeros(8, device="cuda")
    rc = L.msb_rmsnorm_bwd_noalloc(_vp(z), _vp(z), _vp(z), _vp(z), _vp(z), _vp(z), 1, cols, 0, 0, 0,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 2
    assert b"not supported" in L.msb_last_error()
