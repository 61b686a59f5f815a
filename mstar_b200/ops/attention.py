"""Attention over a paged KV pool or dense K/V: prefill, decode (split-KV), DiT/encoder varlen; causal, full and
sliding-window masks; GQA.

GPU path: ``csrc/attention_tcgen05.cu`` (tcgen05 QK^T and PV with TMEM accumulators, TMA page gathers).
CPU path and oracle: ``attention_ref`` (fp32, materialised scores).

KV pool layout of one layer: ``[num_pages, 2, Hkv, page_size, D]`` (K then V, heads before tokens, so a (page,
head) slab is one contiguous TMA box). The reference keeps ``[pages, 2, page_size, Hkv, D]`` and calls
FlashInfer's paged wrappers (mstar/utils/flashinfer_utils.py:70-489, mstar/engine/kv_cache_engine.py:231-235).
"""
from __future__ import annotations

import ctypes
import os
import math
from dataclasses import dataclass

import torch

from . import _lib

_SCRATCH: dict[tuple[int, int], dict] = {}


@dataclass
class AttnPlan:
    """Device-side description of a batch, written by the cache manager before each step (no host work in the
    step itself, so the step can be captured in a CUDA graph)."""
    q_indptr: torch.Tensor          # int32 [B+1]
    kv_lens: torch.Tensor           # int32 [B] (keys visible, including this step's tokens)
    batch: int
    num_q_tokens: int               # T (rows of q)
    num_q_tiles: int                # upper bound of sum ceil(q_len / (128 // G))
    page_indptr: torch.Tensor | None = None   # int32 [B+1]
    page_indices: torch.Tensor | None = None  # int32 [sum pages]
    kv_indptr: torch.Tensor | None = None     # dense mode: int32 [B+1]
    splits: int = 1
    causal: bool = True
    window: int = 0
    max_q_len: int = 0              # largest q_len of the batch when known (1 = plain decode); 0 = unknown


def count_q_tiles(q_lens, group: int) -> int:
    tpt = max(1, 128 // group)
    return int(sum((int(n) + tpt - 1) // tpt for n in q_lens))


def choose_splits(batch: int, num_kv_heads: int, num_q_tiles: int, max_kv_len: int, sm_count: int = 148) -> int:
    """Split-KV factor: fill the SMs when the batch is small and the context is long."""
    forced = os.environ.get("MSTAR_DECODE_SPLITS")
    if forced:
        return max(1, int(forced))
    ctas = max(1, num_q_tiles * num_kv_heads)
    ktiles = max(1, (max_kv_len + 127) // 128)
    if ctas >= sm_count or ktiles <= 2:
        return 1
    return int(max(1, min(sm_count // ctas, ktiles // 2, 32)))


def _scratch(device, rows: int, D: int, splits: int, n_counters: int):
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    s = _SCRATCH.get(key)
    need_o = splits * rows * D
    need_c = n_counters
    if s is None or s["o"].numel() < need_o or s["c"].numel() < need_c:
        s = dict(o=torch.empty(max(need_o, 1 << 20), dtype=torch.float32, device=device),
                 ml=torch.empty(max(splits * rows * 2, 1 << 16), dtype=torch.float32, device=device),
                 c=torch.zeros(max(need_c, 4096), dtype=torch.int32, device=device))
        _SCRATCH[key] = s
    elif s["ml"].numel() < splits * rows * 2:
        s["ml"] = torch.empty(splits * rows * 2, dtype=torch.float32, device=device)
    return s


def reserve_scratch(device, rows: int, D: int, splits: int, n_counters: int) -> None:
    """Allocate split-KV scratch ahead of CUDA-graph capture."""
    _scratch(device, rows, D, splits, n_counters)


def attention_ref(q, plan: AttnPlan, *, kv_cache=None, k=None, v=None, scale=None, lse: bool = False):
    """fp32 oracle. q: [T, Hq, D]."""
    T, Hq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    lse_out = torch.full((T, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    qi = plan.q_indptr.tolist()
    kl = plan.kv_lens.tolist()
    for b in range(plan.batch):
        qs, qe = qi[b], qi[b + 1]
        ql, n = qe - qs, kl[b]
        if ql == 0:
            continue
        if kv_cache is not None:
            ps = kv_cache.shape[3]
            pi = plan.page_indptr.tolist()
            pages = plan.page_indices[pi[b]:pi[b + 1]].long()
            kk = kv_cache[pages, 0].permute(1, 0, 2, 3).reshape(kv_cache.shape[2], -1, D)[:, :n].float()
            vv = kv_cache[pages, 1].permute(1, 0, 2, 3).reshape(kv_cache.shape[2], -1, D)[:, :n].float()
        else:
            ki = plan.kv_indptr.tolist()
            kk = k[ki[b]:ki[b] + n].permute(1, 0, 2).float()
            vv = v[ki[b]:ki[b] + n].permute(1, 0, 2).float()
        Hkv = kk.shape[0]
        G = Hq // Hkv
        qq = q[qs:qe].float().permute(1, 0, 2)                       # [Hq, ql, D]
        kk = kk.repeat_interleave(G, dim=0)
        vv = vv.repeat_interleave(G, dim=0)
        s = torch.matmul(qq, kk.transpose(1, 2)) * scale             # [Hq, ql, n]
        qpos = torch.arange(ql, device=q.device) + (n - ql)
        kpos = torch.arange(n, device=q.device)
        mask = torch.ones(ql, n, dtype=torch.bool, device=q.device)
        if plan.causal:
            mask &= kpos[None, :] <= qpos[:, None]
        if plan.window > 0:
            mask &= kpos[None, :] > (qpos[:, None] - plan.window)
        s = s.masked_fill(~mask[None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        pr = torch.exp(s - l.unsqueeze(-1))
        pr = torch.nan_to_num(pr, nan=0.0)
        out[qs:qe] = torch.matmul(pr, vv).permute(1, 0, 2)
        lse_out[qs:qe] = l.permute(1, 0)
    res = out.to(q.dtype)
    return (res, lse_out) if lse else res


def attention(q: torch.Tensor, plan: AttnPlan, *, kv_cache: torch.Tensor | None = None,
              k: torch.Tensor | None = None, v: torch.Tensor | None = None, scale: float | None = None,
              out: torch.Tensor | None = None, lse: bool = False):
    """q: [T, Hq, D] bf16 (last dim contiguous). Either ``kv_cache`` (paged) or dense ``k``/``v`` [T_kv, Hkv, D]."""
    if not _lib.use_cuda(q):
        return attention_ref(q, plan, kv_cache=kv_cache, k=k, v=v, scale=scale, lse=lse)
    T, Hq, D = q.shape
    if D not in (64, 128):
        if kv_cache is None and D < 128 and q.dtype == torch.bfloat16 and out is None:
            # dense attention with an odd head size (72-wide SigLIP heads, 80-wide ViT heads): zero columns added
            # to q and k leave the scores unchanged and zero columns of v give zero output columns, so the tensor-core
            # kernel runs on the next size it is built for and the padding is cut off again
            Dp = 64 if D < 64 else 128
            pad = (0, Dp - D)
            qp, kp_, vp_ = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
            res = attention(qp, plan, k=kp_, v=vp_, scale=scale if scale is not None else 1.0 / math.sqrt(D), lse=lse)
            if lse:
                return res[0][..., :D].contiguous(), res[1]
            return res[..., :D].contiguous()
        # head sizes the tensor-core kernels are not built for (256-wide Gemma heads, paged caches of odd widths):
        # the fp32 oracle, which is plain tensor code and runs on the GPU too (it reads the plan on the host)
        return attention_ref(q, plan, kv_cache=kv_cache, k=k, v=v, scale=scale, lse=lse)
    assert q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
    paged = kv_cache is not None
    if paged:
        assert kv_cache.is_contiguous() and kv_cache.dtype == torch.bfloat16
        num_pages, _, Hkv, page_size, Dk = kv_cache.shape
        kp, vp, kv_stride, T_kv = kv_cache.data_ptr(), 0, 0, 0
    else:
        assert k.dtype == torch.bfloat16 and k.stride(2) == 1 and k.stride(1) == D and v.stride(1) == D
        assert k.stride(0) == v.stride(0)
        T_kv, Hkv, Dk = k.shape
        num_pages, page_size = 0, 0
        kp, vp, kv_stride = k.data_ptr(), v.data_ptr(), k.stride(0)
    assert Dk == D
    lse_t = torch.empty((T, Hq), dtype=torch.float32, device=q.device) if lse else None
    splits = max(1, int(plan.splits))
    ws_o = ws_ml = cnt = 0
    if splits > 1:
        s = _scratch(q.device, T * Hq, D, splits, max(plan.num_q_tiles, plan.batch) * Hkv)
        ws_o, ws_ml, cnt = s["o"].data_ptr(), s["ml"].data_ptr(), s["c"].data_ptr()
    G = Hq // Hkv
    if paged and D == 128 and 0 < plan.max_q_len and plan.max_q_len * G <= 16:
        # decode: keys on the UMMA M dimension (csrc/attention_decode_tcgen05.cu); no lse output in this path
        if not lse:
            rc = _lib.kernels().mstar_attention_decode(
                ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(out.stride(0)),
                ctypes.c_void_p(plan.q_indptr.data_ptr()), ctypes.c_void_p(plan.kv_lens.data_ptr()),
                int(plan.batch), int(T), int(Hq), int(Hkv), int(D), ctypes.c_void_p(kp), int(num_pages),
                int(page_size), ctypes.c_void_p(plan.page_indptr.data_ptr()),
                ctypes.c_void_p(plan.page_indices.data_ptr()), 1 if plan.causal else 0, int(plan.window),
                ctypes.c_float(scale), splits, int(plan.max_q_len), ctypes.c_void_p(ws_o), ctypes.c_void_p(ws_ml),
                ctypes.c_void_p(cnt), ctypes.c_void_p(_lib.stream_ptr()))
            _lib.check(rc, "mstar_attention_decode")
            return out
    rc = _lib.kernels().mstar_attention(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(out.stride(0)),
        ctypes.c_void_p(plan.q_indptr.data_ptr()), ctypes.c_void_p(plan.kv_lens.data_ptr()),
        int(plan.batch), int(T), int(Hq), int(Hkv), int(D), 1 if paged else 0,
        ctypes.c_void_p(kp), ctypes.c_void_p(vp), ctypes.c_longlong(kv_stride), ctypes.c_longlong(T_kv),
        ctypes.c_void_p(_lib.ptr(plan.kv_indptr)), int(num_pages), int(page_size),
        ctypes.c_void_p(_lib.ptr(plan.page_indptr)), ctypes.c_void_p(_lib.ptr(plan.page_indices)),
        1 if plan.causal else 0, int(plan.window), ctypes.c_float(scale), int(plan.num_q_tiles), splits,
        ctypes.c_void_p(ws_o), ctypes.c_void_p(ws_ml), ctypes.c_void_p(cnt), ctypes.c_void_p(_lib.ptr(lse_t)),
        ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_attention")
    return (out, lse_t) if lse else out


def dense_plan(q_lens, kv_lens, group: int, device, causal: bool = False, window: int = 0) -> AttnPlan:
    """Plan for dense varlen attention: q and k/v are packed request after request."""
    import itertools
    qi = [0] + list(itertools.accumulate(int(x) for x in q_lens))
    ki = [0] + list(itertools.accumulate(int(x) for x in kv_lens))
    return AttnPlan(q_indptr=torch.tensor(qi, dtype=torch.int32, device=device),
                    kv_lens=torch.tensor(list(kv_lens), dtype=torch.int32, device=device),
                    kv_indptr=torch.tensor(ki, dtype=torch.int32, device=device), batch=len(q_lens),
                    num_q_tokens=qi[-1], num_q_tiles=count_q_tiles(q_lens, group), causal=causal, window=window)


def attn_merge_ref(o_a, lse_a, o_b, lse_b):
    m = torch.maximum(lse_a, lse_b)
    safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    ea, eb = torch.exp(lse_a - safe), torch.exp(lse_b - safe)
    den = (ea + eb).clamp_min(1e-38)
    out = o_a.float() * (ea / den)[..., None] + o_b.float() * (eb / den)[..., None]
    return out.to(o_a.dtype), torch.where(torch.isfinite(m), safe + torch.log(den), m)


def attn_merge(o_a: torch.Tensor, lse_a: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor,
               out: torch.Tensor | None = None, lse: bool = False):
    """Combine attention over two disjoint key sets (cached prefix | fresh tokens) from their outputs [T, H, D]
    and log-sum-exps [T, H]. Reference counterpart: the dense-gen path concatenates prefix and fresh K/V before
    one attention call (mstar/engine/cache_manager.py:1455-1485); here the prefix stays paged."""
    if not _lib.use_cuda(o_a):
        o, l = attn_merge_ref(o_a, lse_a, o_b, lse_b)
        return (o, l) if lse else o
    T, H, D = o_a.shape
    assert o_a.is_contiguous() and o_b.is_contiguous() and lse_a.is_contiguous() and lse_b.is_contiguous()
    if out is None:
        out = torch.empty_like(o_a)
    lse_t = torch.empty_like(lse_a) if lse else None
    rc = _lib.kernels().mstar_attn_merge(
        ctypes.c_void_p(o_a.data_ptr()), ctypes.c_void_p(lse_a.data_ptr()), ctypes.c_void_p(o_b.data_ptr()),
        ctypes.c_void_p(lse_b.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(_lib.ptr(lse_t)),
        ctypes.c_longlong(T * H), int(D), ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "mstar_attn_merge")
    return (out, lse_t) if lse else out
