"""Quantisation to fp8 with block scales: eager PyTorch forms, which are also the oracles of the CUDA quantiser
(``msb_quant_1x128`` in csrc/kernels/misc_ops.cu).

  quantize_blockwise(x, block, pow2)          1-D blocks of ``block`` elements, one scale each (optimizer states)
  quant_1x128 / quant_128x128                 activation (per row, 128 along K) and weight (128x128 tiles) scaling of the
                                              "blockwise" fp8 recipe (reference: te/pytorch/fp8/recipes/float8_block_scaling_recipe.py:15-26)
  quant_mx(x, axis)                           MXFP8: blocks of 32 along the reduction axis, e8m0 (power-of-two) scales
                                              (reference: mxfp8_scaling_recipe.py:68-132)
E4M3 max 448, E5M2 max 57344 (reference: te/pytorch/fp8/constants.py:14-58).
"""
from __future__ import annotations

import torch

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def _fmax(dtype):
    return E4M3_MAX if dtype == torch.float8_e4m3fn else E5M2_MAX


def _scale_from_amax(amax, fmax, pow2):
    s = amax.clamp_min(1e-30) / fmax
    if pow2:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    return s


def quantize_blockwise(x, block=128, pow2=False, dtype=torch.float8_e4m3fn):
    n = x.numel()
    pad = (-n) % block
    xf = torch.nn.functional.pad(x.reshape(-1).float(), (0, pad)).view(-1, block)
    scale = _scale_from_amax(xf.abs().amax(dim=1), _fmax(dtype), pow2)
    q = (xf / scale.unsqueeze(1)).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype)
    return q.reshape(-1)[:n + pad], scale


def dequantize_blockwise(q, scale, block=128):
    x = q.float().view(-1, block) * scale.unsqueeze(1)
    return x.reshape(-1)


def quant_1x128(x, dtype=torch.float8_e4m3fn, pow2=False):
    """x [M, K] -> (q [M, K] fp8, scale [M, K/128] fp32): one scale per row per 128 columns."""
    M, K = x.shape
    assert K % 128 == 0
    xf = x.float().view(M, K // 128, 128)
    scale = _scale_from_amax(xf.abs().amax(dim=-1), _fmax(dtype), pow2)
    q = (xf / scale.unsqueeze(-1)).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype).view(M, K)
    return q, scale


def quant_128x128(w, dtype=torch.float8_e4m3fn, pow2=False):
    """w [N, K] -> (q fp8, scale [N/128, K/128])."""
    N, K = w.shape
    assert N % 128 == 0 and K % 128 == 0
    wf = w.float().view(N // 128, 128, K // 128, 128)
    scale = _scale_from_amax(wf.abs().amax(dim=(1, 3)), _fmax(dtype), pow2)
    q = (wf / scale[:, None, :, None]).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype).view(N, K)
    return q, scale


def quant_mx(x, axis=-1, dtype=torch.float8_e4m3fn):
    """MXFP8: blocks of 32 along ``axis`` with e8m0 scales (stored as uint8 exponent + 127)."""
    xt = x.float().movedim(axis, -1)
    shp = xt.shape
    assert shp[-1] % 32 == 0
    xb = xt.reshape(*shp[:-1], shp[-1] // 32, 32)
    scale = _scale_from_amax(xb.abs().amax(dim=-1), _fmax(dtype), True)
    q = (xb / scale.unsqueeze(-1)).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype).reshape(shp).movedim(-1, axis)
    e8m0 = (torch.log2(scale).round().to(torch.int32) + 127).clamp(0, 254).to(torch.uint8)
    return q, e8m0


def dequant_mx(q, e8m0, axis=-1):
    qt = q.float().movedim(axis, -1)
    shp = qt.shape
    s = torch.exp2(e8m0.float() - 127.0)
    return (qt.reshape(*shp[:-1], shp[-1] // 32, 32) * s.unsqueeze(-1)).reshape(shp).movedim(-1, axis)


def fp8_blockwise_matmul_ref(xq, xs, wq, ws, out_dtype=torch.bfloat16):
    """y = x @ w.T from block-quantised operands (xq [M,K], xs [M,K/128]; wq [N,K], ws [N/128,K/128]); fp32 reference."""
    M, K = xq.shape
    N = wq.shape[0]
    x = xq.float().view(M, K // 128, 128) * xs.unsqueeze(-1)
    w = wq.float().view(N // 128, 128, K // 128, 128) * ws[:, None, :, None]
    return (x.view(M, K) @ w.view(N, K).t()).to(out_dtype)
