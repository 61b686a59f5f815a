"""Fused per-head QK RMSNorm + rotary embedding + KV write (into the paged pool and/or dense tensors).

GPU: ``rope_kv_kernel`` in csrc/elementwise.cu. Oracle: ``rope_kv_ref``.
Rotary variants are data, not code: ``inv_freq`` carries plain / llama-3 scaled frequencies, ``axis_of_freq``
selects the position axis of each frequency (interleaved 3-D mRoPE sections), ``interleaved`` picks pairwise
instead of split-half rotation.
Reference counterparts: mstar/utils/attention.py:137-286 (Triton qk-norm+rope, rope), FlashInfer rope calls
(mstar/engine/cache_manager.py:519-528), KV index_put (mstar/utils/flashinfer_utils.py:273-290),
mRoPE (mstar/model/qwen3_omni/components/rope.py:153-200).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib


def make_inv_freq(rot_dim: int, theta: float, device=None, llama3: dict | None = None) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if llama3:
        factor = llama3.get("factor", 8.0)
        lo = llama3.get("low_freq_factor", 1.0)
        hi = llama3.get("high_freq_factor", 4.0)
        orig = llama3.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv
        smooth = (orig / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > orig / lo, inv / factor,
                             torch.where(wavelen < orig / hi, inv, (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    return inv.to(torch.float32).to(device)


def mrope_axis_table(sections: list[int], interleaved: bool = True) -> torch.Tensor:
    """axis (0=t,1=h,2=w) of every rotary frequency. ``interleaved``: t,h,w,t,h,w,... over the first
    3*min-section frequencies then t (Qwen3-Omni style); else contiguous blocks (Qwen2-VL style)."""
    half = sum(sections)
    ax = torch.zeros(half, dtype=torch.int8)
    if interleaved:
        for i in range(half):
            a = i % 3
            if a == 1 and i < 3 * sections[1]:
                ax[i] = 1
            elif a == 2 and i < 3 * sections[2]:
                ax[i] = 2
    else:
        o = 0
        for a, n in enumerate(sections):
            ax[o:o + n] = a
            o += n
    return ax


def rope_kv_ref(qkv, positions, inv_freq, Hq, Hkv, D, *, rot_dim=None, axis_of_freq=None, q_norm_w=None,
                k_norm_w=None, norm_eps=1e-6, interleaved=False, gemma_norm=False, q_scale=1.0):
    """Returns (q [T,Hq,D], k [T,Hkv,D], v [T,Hkv,D]) in qkv.dtype."""
    T = qkv.shape[0]
    rot_dim = rot_dim or D
    half = rot_dim // 2
    q = qkv[:, :Hq * D].reshape(T, Hq, D).float()
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).float()
    v = qkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D].reshape(T, Hkv, D)
    pos = positions.reshape(-1, T).float()
    if axis_of_freq is None:
        p = pos[0][:, None].expand(T, half)
    else:
        p = pos[axis_of_freq.long().to(pos.device)].transpose(0, 1)     # [T, half]
    ang = p * inv_freq.float()[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def one(x, w):
        if w is not None:
            x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + norm_eps) * (w.float() + (1.0 if gemma_norm else 0.0))
            x = x.to(qkv.dtype).float()
        if interleaved:
            x0, x1 = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2]
        else:
            x0, x1 = x[..., :half], x[..., half:rot_dim]
        y0, y1 = x0 * cs - x1 * sn, x1 * cs + x0 * sn
        out = x.clone()
        if interleaved:
            out[..., 0:rot_dim:2], out[..., 1:rot_dim:2] = y0, y1
        else:
            out[..., :half], out[..., half:rot_dim] = y0, y1
        return out
    qo = (one(q, q_norm_w) * q_scale).to(qkv.dtype)
    ko = one(k, k_norm_w).to(qkv.dtype)
    return qo, ko, v.contiguous()


def write_kv_ref(cache, k, v, token_req, cache_pos, page_indptr, page_indices):
    ps = cache.shape[3]
    tr, cp = token_req.tolist(), cache_pos.tolist()
    pi, pidx = page_indptr.tolist(), page_indices.tolist()
    for t in range(k.shape[0]):
        if tr[t] < 0 or cp[t] < 0:
            continue
        page = pidx[pi[tr[t]] + cp[t] // ps]
        cache[page, 0, :, cp[t] % ps] = k[t]
        cache[page, 1, :, cp[t] % ps] = v[t]


def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, Hq: int, Hkv: int, D: int, *,
            rot_dim: int | None = None, axis_of_freq: torch.Tensor | None = None,
            q_norm_w: torch.Tensor | None = None, k_norm_w: torch.Tensor | None = None, norm_eps: float = 1e-6,
            interleaved: bool = False, gemma_norm: bool = False, q_scale: float = 1.0,
            cache: torch.Tensor | None = None, token_req: torch.Tensor | None = None,
            cache_pos: torch.Tensor | None = None, page_indptr: torch.Tensor | None = None,
            page_indices: torch.Tensor | None = None, dense_kv: bool = False,
            q_out: torch.Tensor | None = None):
    """qkv: [T, (Hq+2Hkv)*D]; positions: int32 [T] or [n_axes, T]. Writes K/V into ``cache`` (paged pool of the
    layer) when given; returns (q, k, v) where k, v are dense tensors only when ``dense_kv``."""
    T = qkv.shape[0]
    rot_dim = rot_dim or D
    if not _lib.use_cuda(qkv):
        q, k, v = rope_kv_ref(qkv, positions, inv_freq, Hq, Hkv, D, rot_dim=rot_dim, axis_of_freq=axis_of_freq,
                              q_norm_w=q_norm_w, k_norm_w=k_norm_w, norm_eps=norm_eps, interleaved=interleaved,
                              gemma_norm=gemma_norm, q_scale=q_scale)
        if cache is not None:
            write_kv_ref(cache, k, v, token_req, cache_pos, page_indptr, page_indices)
        return q, (k if dense_kv else None), (v if dense_kv else None)
    assert qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and positions.stride(-1) == 1
    if q_out is None:
        q_out = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
    k_out = v_out = None
    if dense_kv:
        k_out = torch.empty((T, Hkv, D), dtype=qkv.dtype, device=qkv.device)
        v_out = torch.empty((T, Hkv, D), dtype=qkv.dtype, device=qkv.device)
    page_size = cache.shape[3] if cache is not None else 0
    if cache is not None:
        assert token_req.dtype == torch.int32 and cache_pos.dtype == torch.int32
    rc = _lib.kernels().mstar_rope_kv(
        ctypes.c_void_p(qkv.data_ptr()), ctypes.c_longlong(qkv.stride(0)), ctypes.c_void_p(q_out.data_ptr()),
        ctypes.c_void_p(_lib.ptr(k_out)), ctypes.c_void_p(_lib.ptr(v_out)), ctypes.c_void_p(_lib.ptr(cache)),
        ctypes.c_void_p(positions.data_ptr()),
        ctypes.c_longlong(positions.stride(0) if positions.dim() > 1 else T), ctypes.c_void_p(inv_freq.data_ptr()),
        ctypes.c_void_p(_lib.ptr(axis_of_freq)), ctypes.c_void_p(_lib.ptr(q_norm_w)),
        ctypes.c_void_p(_lib.ptr(k_norm_w)), ctypes.c_void_p(_lib.ptr(token_req)),
        ctypes.c_void_p(_lib.ptr(cache_pos)), ctypes.c_void_p(_lib.ptr(page_indptr)),
        ctypes.c_void_p(_lib.ptr(page_indices)), int(T), int(Hq), int(Hkv), int(D), int(rot_dim), int(page_size),
        1 if interleaved else 0, 1 if gemma_norm else 0, ctypes.c_float(norm_eps), ctypes.c_float(q_scale),
        ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_rope_kv")
    return q_out, k_out, v_out
