"""RMSNorm / LayerNorm with fused residual add and AdaLN-style modulation.

GPU: ``norm_kernel`` in csrc/elementwise.cu. Oracle: ``norm_ref``.
Reference counterparts: Triton rms_norm (mstar/utils/attention.py:447-501), FlashInfer rmsnorm
(mstar/utils/flashinfer_utils.py:25-50, mstar/model/components/norm.py:22-62), adaptive RMSNorm
(mstar/utils/adarms_norm.py:31-77), Wan2.2 AdaLN modulation (mstar/model/wan22/components/dit.py:254-272).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def norm_ref(x, weight=None, eps=1e-6, residual=None, bias=None, scale=None, shift=None, layernorm=False,
             gemma=False):
    """Returns (y, new_residual). new_residual is None when no residual was given."""
    h = x.float()
    new_res = None
    if residual is not None:
        new_res = (h + residual.float()).to(x.dtype)
        h = new_res.float()
    if layernorm:
        mu = h.mean(-1, keepdim=True)
        var = ((h - mu) ** 2).mean(-1, keepdim=True)
        y = (h - mu) * torch.rsqrt(var + eps)
    else:
        y = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * (weight.float() + (1.0 if gemma else 0.0))
    if bias is not None:
        y = y + bias.float()
    if scale is not None:
        # scale/shift: [n_mod, hidden]; rows are grouped evenly over the modulation rows
        rows = y.reshape(-1, y.shape[-1]).shape[0]
        n_mod = scale.reshape(-1, scale.shape[-1]).shape[0]
        rpm = rows // n_mod
        sc = scale.reshape(n_mod, -1).float().repeat_interleave(rpm, 0).reshape(y.shape)
        sh = shift.reshape(n_mod, -1).float().repeat_interleave(rpm, 0).reshape(y.shape)
        y = y * (1 + sc) + sh
    return y.to(x.dtype), new_res


def norm(x: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-6, *,
         residual: torch.Tensor | None = None, bias: torch.Tensor | None = None,
         scale: torch.Tensor | None = None, shift: torch.Tensor | None = None, layernorm: bool = False,
         gemma: bool = False, out: torch.Tensor | None = None):
    """y = norm(x + residual) * weight (+bias) [* (1 + scale) + shift]; returns (y, x + residual or None).
    With a residual the sum is written back into ``residual`` in place (and returned)."""
    if not _lib.use_cuda(x):
        y, nr = norm_ref(x, weight, eps, residual, bias, scale, shift, layernorm, gemma)
        if residual is not None:
            residual.copy_(nr)
            nr = residual
        if out is not None:
            out.copy_(y.reshape(out.shape))
            y = out
        return y, nr
    assert x.dtype == torch.bfloat16
    hidden = x.shape[-1]
    x2 = x.reshape(-1, hidden)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    if out is None:
        out = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    out2 = out.reshape(-1, hidden)
    res2 = None
    if residual is not None:
        assert residual.is_contiguous() or residual.stride(-1) == 1
        res2 = residual.reshape(-1, hidden)
    n_mod, mod_stride, rpm = 0, 0, 1
    if scale is not None:
        sc2, sh2 = scale.reshape(-1, hidden), shift.reshape(-1, hidden)
        assert sc2.stride(-1) == 1 and sh2.stride(-1) == 1 and sc2.stride(0) == sh2.stride(0)
        n_mod = sc2.shape[0]
        mod_stride = sc2.stride(0)
        rpm = rows // n_mod
        scale, shift = sc2, sh2
    rc = _lib.kernels().mstar_norm(
        ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(_lib.ptr(res2)), ctypes.c_void_p(_lib.ptr(res2)),
        ctypes.c_void_p(_lib.ptr(weight)), ctypes.c_void_p(_lib.ptr(bias)), ctypes.c_void_p(_lib.ptr(scale)),
        ctypes.c_void_p(_lib.ptr(shift)), ctypes.c_void_p(out2.data_ptr()), int(rows), int(hidden),
        ctypes.c_longlong(x2.stride(0)), ctypes.c_longlong(res2.stride(0) if res2 is not None else 0),
        ctypes.c_longlong(out2.stride(0)), int(rpm), ctypes.c_longlong(mod_stride), ctypes.c_float(eps),
        1 if layernorm else 0, 1 if gemma else 0, ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_norm")
    return out.reshape(x.shape), residual


def rms_norm(x, weight, eps=1e-6, residual=None, gemma=False):
    return norm(x, weight, eps, residual=residual, gemma=gemma)
