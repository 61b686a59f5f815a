"""Dense projections: ``y = x @ w.T (+bias) (+residual)`` with optional SwiGLU / GELU epilogue.

GPU path: the hand-written tcgen05 kernel of ``csrc/gemm_tcgen05.cu`` (TMEM accumulators, TMA-fed, split-K
through a scratch workspace for skinny decode shapes). CPU path and test oracle: ``linear_ref`` in fp32.

Reference counterpart: cuBLAS through ``F.linear`` in mstar/model/components/distributed/linear.py:8-419 and
mstar/model/components/mlp.py (SwiGLU is a separate elementwise op there).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

EPILOGUE_NONE = 0
EPILOGUE_SWIGLU = 1   # weight rows interleave (gate_j, up_j); output has N/2 columns
EPILOGUE_GELU = 2

_WORKSPACES: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
WORKSPACE_BYTES = 96 << 20
N_COUNTERS = 1 << 16


def workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Split-K scratch (fp32 partial tiles) and per-tile arrival counters for the current stream.
    One pair per (device, stream) so that kernels on different streams never share scratch."""
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = (torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=device),
              torch.zeros(N_COUNTERS, dtype=torch.int32, device=device))
        _WORKSPACES[key] = ws
    return ws


def interleave_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """Stack gate and up projection weights row-interleaved: row 2j = gate_j, row 2j+1 = up_j, which is the
    layout the SwiGLU epilogue expects (the pair lands in neighbouring accumulator columns / lanes)."""
    assert gate_w.shape == up_w.shape
    out = torch.stack([gate_w, up_w], dim=1)
    return out.reshape(2 * gate_w.shape[0], *gate_w.shape[1:]).contiguous()


def split_gate_up(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of ``interleave_gate_up``: (gate rows, up rows)."""
    return w[0::2].contiguous(), w[1::2].contiguous()


class PackedWeight:
    """A [N, K] bf16 weight stored tile by tile for streaming: ``[ceil(N/128)][ceil(K/64)]`` tiles of 128 rows x 64
    columns, each 16 KB contiguous, zero-padded at the ragged edges. One TMA box of the GEMM kernels is then one
    contiguous run in DRAM instead of 128 separate 128-byte pieces a row pitch apart. ``linear`` accepts it in place
    of the plain weight on CUDA; ``unpack`` gives the plain matrix back."""

    __slots__ = ("data", "shape")

    def __init__(self, data: torch.Tensor, shape: tuple[int, int]):
        self.data, self.shape = data, tuple(shape)

    @property
    def device(self):
        return self.data.device

    @property
    def dtype(self):
        return self.data.dtype

    def unpack(self) -> torch.Tensor:
        N, K = self.shape
        tn, tk = (N + 127) // 128, (K + 63) // 64
        w = self.data.view(tn, tk, 128, 64).permute(0, 2, 1, 3).reshape(tn * 128, tk * 64)
        return w[:N, :K].contiguous()


def pack_weight(w: torch.Tensor) -> PackedWeight:
    assert w.dim() == 2 and w.dtype == torch.bfloat16
    N, K = w.shape
    tn, tk = (N + 127) // 128, (K + 63) // 64
    wp = F.pad(w, (0, tk * 64 - K, 0, tn * 128 - N)) if (N % 128 or K % 64) else w
    data = wp.view(tn, 128, tk, 64).permute(0, 2, 1, 3).contiguous().view(tn * tk * 128, 64)
    return PackedWeight(data, (N, K))


def linear_ref(x, w, bias=None, residual=None, epilogue=EPILOGUE_NONE, out_dtype=None, out_scale=1.0):
    """fp32 PyTorch oracle with the same rounding points as the kernel (one rounding at the output)."""
    out_dtype = out_dtype or x.dtype
    y = F.linear(x.float(), w.float()) * out_scale
    if bias is not None:
        y = y + bias.float()
    if epilogue == EPILOGUE_SWIGLU:
        g, u = y[..., 0::2], y[..., 1::2]
        y = F.silu(g) * u
    elif epilogue == EPILOGUE_GELU:
        y = F.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype)


def gemm_plan(M: int, N: int, K: int) -> dict:
    lib = _lib.kernels()
    swap, bn, splits, tiles = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    ws = ctypes.c_longlong()
    lib.mstar_gemm_plan(M, N, K, ctypes.byref(swap), ctypes.byref(bn), ctypes.byref(splits), ctypes.byref(ws),
                        ctypes.byref(tiles))
    return dict(swap=swap.value, bn=bn.value, splits=splits.value, ws_bytes=ws.value, tiles=tiles.value)


class FoldedNorm:
    """RMSNorms folded into one projection of a decode step (see ``mstar_gemm_norm_hint``).

    ``ss_in``:  fp32 [rows] sums of squares of the activation rows: the projection's weight already carries the norm's
                gain, the kernel multiplies output row t by ``rsqrt(ss_in[t] / hidden + eps)``.
    ``ss_out``: fp32 [rows] accumulator that receives the sums of squares of the bf16 output rows (the new residual
                stream); must be zero when the kernel runs.
    ``ss_zero``: an accumulator that this kernel clears for the next producer (nobody reads it any more by then).
    """

    def __init__(self, hidden: int, eps: float, ss_in=None, ss_out=None, ss_zero=None):
        self.hidden, self.eps, self.ss_in, self.ss_out, self.ss_zero = hidden, eps, ss_in, ss_out, ss_zero

    def arm(self) -> None:
        _lib.kernels().mstar_gemm_norm_hint(
            ctypes.c_void_p(_lib.ptr(self.ss_in)), ctypes.c_void_p(_lib.ptr(self.ss_out)),
            ctypes.c_void_p(_lib.ptr(self.ss_zero)), int(self.ss_zero.numel()) if self.ss_zero is not None else 0,
            ctypes.c_float(1.0 / self.hidden), ctypes.c_float(self.eps))

    def linear_ref(self, x, w, bias, residual, epilogue, out):
        """The same arithmetic in PyTorch (CPU path and test oracle)."""
        x2 = x.reshape(-1, x.shape[-1])
        rows = x2.shape[0]
        y = x2.float() @ w.float().t()
        if self.ss_in is not None:
            y = y * torch.rsqrt(self.ss_in[:rows].float() / self.hidden + self.eps)[:, None]
        if bias is not None:
            y = y + bias.float()
        if epilogue == EPILOGUE_SWIGLU:
            y = F.silu(y[:, 0::2]) * y[:, 1::2]
        elif epilogue == EPILOGUE_GELU:
            y = F.gelu(y, approximate="tanh")
        if residual is not None:
            y = y + residual.reshape(rows, -1).float()
        y = y.to(x.dtype)
        if self.ss_zero is not None:
            self.ss_zero.zero_()
        if self.ss_out is not None:
            self.ss_out[:rows] += (y.float() ** 2).sum(-1)
        if out is not None:
            out.reshape(rows, -1).copy_(y)
            return out
        return y.reshape(*x.shape[:-1], y.shape[-1])


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, epilogue: int = EPILOGUE_NONE,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
           out_scale: float = 1.0, force_splits: int = 0, norm: "FoldedNorm | None" = None) -> torch.Tensor:
    """x: [..., K], w: [N, K] (or a ``PackedWeight``) -> [..., N] (N/2 for the SwiGLU epilogue).
    ``norm``: RMSNorms folded into this projection (``FoldedNorm``; decode sizes, at most 128 rows)."""
    packed = isinstance(w, PackedWeight)
    if packed and not _lib.use_cuda(x, w.data):
        w, packed = w.unpack(), False
    if not packed and not _lib.use_cuda(x, w):
        if norm is not None:
            return norm.linear_ref(x, w, bias, residual, epilogue, out)
        return linear_ref(x, w, bias, residual, epilogue, out_dtype, out_scale)
    if norm is not None:
        assert x.numel() // x.shape[-1] <= 128 and (out_dtype in (None, torch.bfloat16)), "folded norms are a decode-size path"
        norm.arm()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "tcgen05 GEMM takes bf16 operands"
    K = x.shape[-1]
    N = w.shape[0]
    assert w.shape[1] == K
    if packed:
        assert K % 8 == 0, "packed weights need K % 8 == 0"
        if x.numel() // K > 128 and N <= 128:
            w, packed = w.unpack(), False      # the token-major kernel has no packed path for tiles under 128 rows
    if not packed and (K % 8 or (N % 8 and N * K <= (1 << 22))) and epilogue != EPILOGUE_SWIGLU and residual is None and out is None:
        # odd widths (a 7-wide action vector, a 10-wide head): zero-pad to the 16-byte granularity of the TMA tiles.
        # Only small weights are padded on the fly (a copy per call); a large matrix with an odd row COUNT runs as
        # it is (the kernel handles a ragged last tile), and an odd row LENGTH should be padded once at load time.
        pk, pn = (-K) % 8, ((-N) % 8 if N * K <= (1 << 22) else 0)
        xp = F.pad(x.reshape(-1, K), (0, pk))
        wp = F.pad(w, (0, pk, 0, pn))
        bp = F.pad(bias, (0, pn)) if bias is not None else None
        y = linear(xp, wp, bp, None, epilogue, out_dtype, None, out_scale, force_splits)
        return y[:, :N].reshape(*x.shape[:-1], N)
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if not packed and (w.stride(-1) != 1 or w.stride(0) % 8):
        w = w.contiguous()
    wt = w.data if packed else w
    M = x2.shape[0]
    n_out = N // 2 if epilogue == EPILOGUE_SWIGLU else N
    out_dtype = out_dtype or x.dtype
    assert out_dtype in (torch.bfloat16, torch.float32)
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    else:
        assert out.dtype == out_dtype and out.stride(-1) == 1
    out2 = out.reshape(-1, n_out) if out.dim() != 2 else out
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, n_out)
        assert res2.dtype == torch.bfloat16 and res2.stride(-1) == 1
    if M == 0:
        return out.reshape(*x.shape[:-1], n_out)
    ws, counters = workspace(x.device)
    rc = _lib.kernels().mstar_gemm_bf16(
        ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(wt.data_ptr()), ctypes.c_void_p(out2.data_ptr()),
        M, N, K, x2.stride(0), wt.stride(0), out2.stride(0),
        ctypes.c_void_p(_lib.ptr(bias)), ctypes.c_void_p(_lib.ptr(res2)),
        res2.stride(0) if res2 is not None else 0, int(epilogue), 1 if out_dtype == torch.float32 else 0,
        ctypes.c_float(out_scale), ctypes.c_void_p(ws.data_ptr()), ctypes.c_longlong(ws.numel()),
        ctypes.c_void_p(counters.data_ptr()), counters.numel(), int(force_splits), 1 if packed else 0,
        ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_gemm_bf16")
    return out.reshape(*x.shape[:-1], n_out)
