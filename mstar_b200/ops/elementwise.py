"""Small fused elementwise ops: SiLU/GELU-mul, embedding gather, gated residual, CFG combine + Euler step,
affine image normalise, device-side decode-state advance.

GPU: csrc/elementwise.cu. Oracles: the ``*_ref`` functions.
Reference counterparts: Triton act_and_mul (mstar/utils/fused_moe/kernels.py:244-298), vocab-parallel embedding
(mstar/model/components/distributed/embedding.py:27-116), BAGEL CFG combine + renorm + Euler
(mstar/model/bagel/submodules.py:1005-1100), Pi0.5 image normalise (mstar/model/pi05/kernels/image_normalize.py:39).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib


def act_mul_ref(x, act="silu"):
    I = x.shape[-1] // 2
    g, u = x[..., :I].float(), x[..., I:].float()
    a = F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")
    return (a * u).to(x.dtype)


def act_mul(x: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """x: [..., 2I] (gate half then up half) -> act(gate) * up."""
    if not _lib.use_cuda(x):
        return act_mul_ref(x, act)
    I = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * I).contiguous()
    out = torch.empty((x2.shape[0], I), dtype=x.dtype, device=x.device)
    rc = _lib.kernels().mstar_act_mul(ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                      ctypes.c_longlong(x2.shape[0]), int(I), 0 if act == "silu" else 1,
                                      ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_act_mul")
    return out.reshape(*x.shape[:-1], I)


def embed_ref(ids, table, vocab_start=0, scale=1.0):
    V = table.shape[0]
    ok = (ids >= vocab_start) & (ids < vocab_start + V)
    rows = table[(ids - vocab_start).clamp(0, V - 1)]
    rows = torch.where(ok[..., None], rows, torch.zeros_like(rows))
    return (rows.float() * scale).to(table.dtype) if scale != 1.0 else rows


def embed(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0, scale: float = 1.0,
          out: torch.Tensor | None = None) -> torch.Tensor:
    """Row gather; ids outside [vocab_start, vocab_start + rows) give zero rows (vocab-parallel shards)."""
    if not _lib.use_cuda(table):
        return embed_ref(ids, table, vocab_start, scale)
    assert ids.dtype == torch.int64 and table.dtype == torch.bfloat16 and table.is_contiguous()
    flat = ids.reshape(-1).contiguous()
    T, H = flat.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    rc = _lib.kernels().mstar_embed_gather(ctypes.c_void_p(flat.data_ptr()), ctypes.c_void_p(table.data_ptr()),
                                           ctypes.c_void_p(out.data_ptr()), int(T), int(H),
                                           ctypes.c_longlong(vocab_start),
                                           ctypes.c_longlong(vocab_start + table.shape[0]), ctypes.c_float(scale),
                                           ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_embed_gather")
    return out.reshape(*ids.shape, H)


def gated_residual_ref(x, y, gate=None):
    if gate is None:
        return (x.float() + y.float()).to(x.dtype)
    rows = x.reshape(-1, x.shape[-1]).shape[0]
    g = gate.reshape(-1, gate.shape[-1]).float()
    g = g.repeat_interleave(rows // g.shape[0], 0).reshape(x.shape)
    return (x.float() + g * y.float()).to(x.dtype)


def gated_residual(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
    """x + gate * y, gate rows [n_mod, hidden] spread evenly over the rows of x."""
    if not _lib.use_cuda(x):
        return gated_residual_ref(x, y, gate)
    H = x.shape[-1]
    x2, y2 = x.reshape(-1, H).contiguous(), y.reshape(-1, H).contiguous()
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    rpm, gs = 1, 0
    if gate is not None:
        gate = gate.reshape(-1, H)
        assert gate.stride(-1) == 1
        rpm, gs = rows // gate.shape[0], gate.stride(0)
    rc = _lib.kernels().mstar_gated_residual(ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(y2.data_ptr()),
                                             ctypes.c_void_p(_lib.ptr(gate)), ctypes.c_void_p(out.data_ptr()),
                                             ctypes.c_longlong(rows), int(H), int(rpm), ctypes.c_longlong(gs),
                                             ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_gated_residual")
    return out.reshape(x.shape)


def cfg_combine_ref(v_cond, v_uncond, x, dt, s_text, *, v_img=None, s_img=1.0, renorm=False, renorm_min=0.0):
    c, u = v_cond.float(), v_uncond.float()
    if v_img is not None:
        t = u + s_text * (c - u)
        v = v_img.float() + s_img * (t - v_img.float())
    else:
        v = u + s_text * (c - u)
    if renorm:
        nc = c.norm(dim=-1, keepdim=True)
        nv = v.norm(dim=-1, keepdim=True)
        v = v * (nc / (nv + 1e-8)).clamp(min=renorm_min, max=1.0)
    return x.float() + dt * v, v


def cfg_combine(v_cond, v_uncond, x, dt: float, s_text: float, *, v_img=None, s_img: float = 1.0,
                renorm: bool = False, renorm_min: float = 0.0):
    """Guidance combine + per-row renorm + Euler step on fp32 [rows, cols] tensors -> (x_next, v)."""
    if not _lib.use_cuda(x):
        return cfg_combine_ref(v_cond, v_uncond, x, dt, s_text, v_img=v_img, s_img=s_img, renorm=renorm,
                               renorm_min=renorm_min)
    cols = x.shape[-1]
    f = lambda t: None if t is None else t.reshape(-1, cols).float().contiguous()
    vc, vu, vi, x2 = f(v_cond), f(v_uncond), f(v_img), f(x)
    x_next, v_out = torch.empty_like(x2), torch.empty_like(x2)
    rc = _lib.kernels().mstar_cfg_combine(ctypes.c_void_p(vc.data_ptr()), ctypes.c_void_p(vu.data_ptr()),
                                          ctypes.c_void_p(_lib.ptr(vi)), ctypes.c_void_p(x2.data_ptr()),
                                          ctypes.c_void_p(x_next.data_ptr()), ctypes.c_void_p(v_out.data_ptr()),
                                          int(x2.shape[0]), int(cols), ctypes.c_float(s_text), ctypes.c_float(s_img),
                                          ctypes.c_float(dt), 1 if renorm else 0, ctypes.c_float(renorm_min),
                                          ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_cfg_combine")
    return x_next.reshape(x.shape), v_out.reshape(x.shape)


def affine(x: torch.Tensor, a: float, b: float, out_dtype=torch.bfloat16) -> torch.Tensor:
    """out = x * a + b (image range normalisation)."""
    if not _lib.use_cuda(x):
        return (x.float() * a + b).to(out_dtype)
    xf = x.float().contiguous()
    out = torch.empty(xf.shape, dtype=out_dtype, device=x.device)
    bf = out_dtype == torch.bfloat16
    rc = _lib.kernels().mstar_affine(ctypes.c_void_p(xf.data_ptr()), ctypes.c_void_p(out.data_ptr() if bf else 0),
                                     ctypes.c_void_p(0 if bf else out.data_ptr()), ctypes.c_longlong(xf.numel()),
                                     ctypes.c_float(a), ctypes.c_float(b), ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_affine")
    return out


def advance_decode(kv_lens, positions, cache_pos=None, input_ids=None, sampled=None, active=None):
    """One decode step forward on the device: kv_lens += 1, positions (all axes) += 1, cache_pos += 1,
    input_ids = sampled. Entries with kv_lens == 0 (padding) or active == 0 keep their plan."""
    B = kv_lens.numel()
    pos2 = positions if positions.dim() > 1 else positions.reshape(1, B)
    if not _lib.use_cuda(kv_lens):
        m = kv_lens > 0
        if active is not None:
            m &= active.bool()
        if input_ids is not None and sampled is not None:
            input_ids.copy_(sampled)
        kv_lens[m] += 1
        pos2[:, m] += 1
        if cache_pos is not None:
            cache_pos[m] += 1
        return
    assert pos2.stride(1) == 1
    rc = _lib.kernels().mstar_advance_decode(ctypes.c_void_p(kv_lens.data_ptr()), ctypes.c_void_p(positions.data_ptr()),
                                             ctypes.c_void_p(_lib.ptr(cache_pos)), ctypes.c_void_p(_lib.ptr(input_ids)),
                                             ctypes.c_void_p(_lib.ptr(sampled)), ctypes.c_void_p(_lib.ptr(active)),
                                             int(B), int(pos2.shape[0]), int(pos2.stride(0)),
                                             ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_advance_decode")


def snake_ref(x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    a = alpha.reshape(1, -1, 1).float()
    xf = x.float()
    return (xf + torch.sin(a * xf).pow(2) / (a + 1e-9)).to(x.dtype)


def snake(x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """Snake activation y = x + sin^2(alpha x) / alpha on [B, C, T] (alpha per channel), one fused kernel on the GPU.
    Reference counterpart: Snake1d of the SNAC decoder (mstar/model/orpheus/components/snac.py:43), composed there
    from separate elementwise ops."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16):
        return snake_ref(x, alpha)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    a = alpha.reshape(-1).float().contiguous()
    B, C, T = xc.shape
    rc = _lib.kernels().mstar_snake(ctypes.c_void_p(xc.data_ptr()), ctypes.c_void_p(a.data_ptr()),
                                    ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(xc.numel()), int(C),
                                    ctypes.c_longlong(T), 1 if x.dtype == torch.float32 else 0,
                                    ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_snake")
    return out
