"""Block-scaled fp8 (e4m3) projections: 1 x 128 activation scales, 128 x 128 weight scales, fp32 accumulation,
bf16 output. ``y = (x8 * a_scale) @ (w8 * w_scale).T`` with the scales applied per 128-wide K block.

GPU path: ``gemm_fp8_blockscaled_kernel`` of ``csrc/gemm_tcgen05.cu`` (kind::f8f6f4 UMMAs, one K block per TMEM
accumulator buffer, scales applied by the epilogue warps) and ``quant_fp8_1x128_kernel`` of ``csrc/elementwise.cu``.
CPU path and test oracle: the same arithmetic in fp32 PyTorch on de-quantised operands.

The reference serves bf16 only (its fused MoE source carries a note that the fp8 paths were stripped:
mstar/utils/fused_moe/kernels.py:5); this is the fp8 variant of the same projections and expert GEMMs.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import EPILOGUE_GELU, EPILOGUE_NONE, EPILOGUE_SWIGLU

FP8_MAX = 448.0
BLOCK = 128


class Fp8Weight:
    """e4m3 weight [N, K] (or stacked [E, N, K]) with one fp32 scale per 128 x 128 block."""

    __slots__ = ("data", "scale", "shape")

    def __init__(self, data: torch.Tensor, scale: torch.Tensor):
        self.data, self.scale, self.shape = data, scale, tuple(data.shape)

    @property
    def device(self):
        return self.data.device

    def dequant(self) -> torch.Tensor:
        *lead, N, K = self.shape
        s = self.scale.repeat_interleave(BLOCK, dim=-2).repeat_interleave(BLOCK, dim=-1)[..., :N, :K]
        return self.data.float() * s


def quantize_weight(w: torch.Tensor) -> Fp8Weight:
    """[.., N, K] float -> e4m3 with 128 x 128 block scales (scale = max|block| / 448)."""
    *lead, N, K = w.shape
    tn, tk = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    wp = F.pad(w.float(), (0, tk * BLOCK - K, 0, tn * BLOCK - N))
    blocks = wp.reshape(*lead, tn, BLOCK, tk, BLOCK)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-12)             # [.., tn, tk]
    scale = amax / FP8_MAX
    q = (blocks / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.reshape(*lead, tn * BLOCK, tk * BLOCK)[..., :N, :K].contiguous().to(torch.float8_e4m3fn)
    return Fp8Weight(q, scale.contiguous())


def quantize_act_ref(x: torch.Tensor):
    """[M, K] -> (e4m3 [M, K], scale_t fp32 [ceil(K/128), M])."""
    M, K = x.shape
    tk = (K + BLOCK - 1) // BLOCK
    xp = F.pad(x.float(), (0, tk * BLOCK - K)).reshape(M, tk, BLOCK)
    scale = xp.abs().amax(-1).clamp_min(1e-12) / FP8_MAX                 # [M, tk]
    q = (xp / scale[..., None]).reshape(M, tk * BLOCK)[:, :K].contiguous().to(torch.float8_e4m3fn)
    return q, scale.t().contiguous()


def quantize_act(x: torch.Tensor, src_row: torch.Tensor | None = None, src_div: int = 1, rows: int | None = None):
    """Quantise the rows of ``x`` [M, K] bf16. With ``src_row`` (int32), output row r is taken from input row
    ``src_row[r] // src_div`` (negative: a zero row). Returns (e4m3 [rows, K], scale_t [ceil(K/128), ld]) where ld is
    the row count rounded up to 128 (the GEMM's token tile)."""
    M, K = x.shape
    R = rows if rows is not None else (src_row.numel() if src_row is not None else M)
    if not _lib.use_cuda(x):
        if src_row is not None:
            idx = torch.div(src_row.long(), src_div, rounding_mode="floor")
            xs = torch.where((src_row >= 0)[:, None], x[idx.clamp_min(0)], torch.zeros((), dtype=x.dtype))
        else:
            xs = x
        q, st = quantize_act_ref(xs)
        ld = (R + BLOCK - 1) // BLOCK * BLOCK
        return q, F.pad(st, (0, ld - R))
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1 and K % 16 == 0
    tk = (K + BLOCK - 1) // BLOCK
    ld = (R + BLOCK - 1) // BLOCK * BLOCK
    q = torch.empty((R, K), dtype=torch.float8_e4m3fn, device=x.device)
    st = torch.zeros((tk, ld), dtype=torch.float32, device=x.device)
    rc = _lib.kernels().mstar_quant_fp8_1x128(
        ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(x.stride(0)), ctypes.c_void_p(_lib.ptr(src_row)), int(src_div),
        ctypes.c_void_p(q.data_ptr()), ctypes.c_longlong(K), ctypes.c_void_p(st.data_ptr()), int(ld), int(R), int(K),
        ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_quant_fp8_1x128")
    return q, st


def _dequant_act(q: torch.Tensor, scale_t: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    s = scale_t[:, :M].t().repeat_interleave(BLOCK, dim=1)[:, :K]
    return q.float() * s


def linear_fp8_ref(x, w: Fp8Weight, bias=None, residual=None, epilogue=EPILOGUE_NONE, out_dtype=torch.bfloat16):
    """fp32 oracle: quantise the activation the same way, multiply the de-quantised operands."""
    x2 = x.reshape(-1, x.shape[-1])
    q, st = quantize_act_ref(x2)
    y = F.linear(_dequant_act(q, st), w.dequant())
    if bias is not None:
        y = y + bias.float()
    if epilogue == EPILOGUE_SWIGLU:
        y = F.silu(y[..., 0::2]) * y[..., 1::2]
    elif epilogue == EPILOGUE_GELU:
        y = F.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual.reshape(y.shape).float()
    return y.to(out_dtype).reshape(*x.shape[:-1], y.shape[-1])


def linear_fp8(x: torch.Tensor, w: Fp8Weight, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
               epilogue: int = EPILOGUE_NONE, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """x [..., K] bf16, w e4m3 [N, K] -> [..., N] (N/2 with the SwiGLU epilogue over interleaved gate/up rows)."""
    if not _lib.use_cuda(x, w.data):
        return linear_fp8_ref(x, w, bias, residual, epilogue, out_dtype)
    N, K = w.shape
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    n_out = N // 2 if epilogue == EPILOGUE_SWIGLU else N
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    if M == 0:
        return out.reshape(*x.shape[:-1], n_out)
    q, st = quantize_act(x2)
    res2 = residual.reshape(-1, n_out) if residual is not None else None
    rc = _lib.kernels().mstar_gemm_fp8(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(st.data_ptr()), int(st.stride(0)),
        ctypes.c_void_p(w.data.data_ptr()), ctypes.c_void_p(w.scale.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        M, N, K, K, K, out.stride(0), ctypes.c_void_p(_lib.ptr(bias)), ctypes.c_void_p(_lib.ptr(res2)),
        res2.stride(0) if res2 is not None else 0, int(epilogue), 1 if out_dtype == torch.float32 else 0,
        ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_gemm_fp8")
    return out.reshape(*x.shape[:-1], n_out)
