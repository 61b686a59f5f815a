"""Mixture-of-experts ops: routing (softmax / top-k / renorm), expert-sorted alignment, grouped tcgen05 GEMMs with
the SwiGLU epilogue, weighted un-permute; and the expert-parallel variant whose dispatch and combine are peer
stores over the symmetric heap.

GPU: csrc/moe.cu + the grouped mode of csrc/gemm_tcgen05.cu. Oracle: ``moe_ref`` (dense loop over experts, fp32).
Reference counterparts: ``fused_experts`` / ``moe_align_block_size`` (mstar/utils/fused_moe/*), TP-MoE block
(mstar/model/components/moe.py:378-591). The reference has no expert parallelism and no fp8 path; here expert
weights given as ``gemm_fp8.Fp8Weight`` run the block-scaled e4m3 grouped GEMM.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib, gemm, gemm_fp8


def route_ref(logits: torch.Tensor, top_k: int, renorm: bool = True):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, top_k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def moe_ref(x, router_w, w13, w2, top_k, renorm=True, shared=None):
    """x [T,H]; router_w [E,H]; w13 [E, 2I, H] (gate/up rows interleaved); w2 [E, H, I]. fp32 math."""
    T, H = x.shape
    logits = F.linear(x.float(), router_w.float())
    ids, w = route_ref(logits, top_k, renorm)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(w13.shape[0]):
        m = (ids == e)
        rows = m.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        xe = x[rows].float()
        gu = F.linear(xe, w13[e].float())
        h = (F.silu(gu[:, 0::2]) * gu[:, 1::2]).to(x.dtype).float()
        y = F.linear(h, w2[e].float()).to(x.dtype).float()
        wt = (w * m)[rows].sum(-1, keepdim=True)
        out[rows] += wt * y
    return out.to(x.dtype)


def choose_block_rows(n_pairs: int, E: int) -> int:
    avg = max(1, n_pairs // max(1, E))
    for b in (16, 32, 64, 128):
        if avg <= b:
            return b
    return 128


class MoeWorkspace:
    """Device buffers for one MoE call shape (fixed addresses: capturable)."""

    def __init__(self, device, T: int, top_k: int, E_local: int, H: int, I: int, block_rows: int):
        n = T * top_k
        cap = ((n + E_local * (block_rows - 1)) + block_rows - 1) // block_rows * block_rows
        self.T, self.top_k, self.block_rows, self.capacity = T, top_k, block_rows, cap
        d, i32, f32, bf = device, torch.int32, torch.float32, torch.bfloat16
        self.topk_ids = torch.empty(T, top_k, dtype=i32, device=d)
        self.topk_w = torch.empty(T, top_k, dtype=f32, device=d)
        self.sorted_pair = torch.empty(cap, dtype=i32, device=d)
        self.sorted_w = torch.empty(cap, dtype=f32, device=d)
        self.pos_of_pair = torch.empty(n, dtype=i32, device=d)
        self.block_expert = torch.zeros(cap // block_rows, dtype=i32, device=d)
        self.num_blocks = torch.zeros(1, dtype=i32, device=d)
        self.x_sorted = torch.zeros(cap, H, dtype=bf, device=d)
        self.h_sorted = torch.empty(cap, I, dtype=bf, device=d)
        self.y_sorted = torch.empty(cap, H, dtype=bf, device=d)


_WS: dict = {}


def _workspace(device, T, top_k, E_local, H, I, block_rows) -> MoeWorkspace:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, T, top_k, E_local, H, I, block_rows)
    ws = _WS.get(key)
    if ws is None:
        ws = MoeWorkspace(device, T, top_k, E_local, H, I, block_rows)
        _WS[key] = ws
    return ws


def _p(t):
    return ctypes.c_void_p(_lib.ptr(t))


def fused_moe(x: torch.Tensor, router_logits: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, top_k: int,
              renorm: bool = True, expert_range: tuple[int, int] | None = None, add: torch.Tensor | None = None):
    """x [T,H] bf16; router_logits [T,E] fp32; w13 [E_local, 2I, H] (gate/up interleaved); w2 [E_local, H, I].
    ``expert_range`` = (begin, end) global ids of the local experts (TP-MoE / EP shards); pairs routed elsewhere
    contribute nothing. ``add`` is added to the result (shared expert / residual)."""
    T, H = x.shape
    E = router_logits.shape[1]
    E_local, I = w13.shape[0], w2.shape[2]
    e0, e1 = expert_range or (0, E)
    fp8 = isinstance(w13, gemm_fp8.Fp8Weight)
    if fp8 and not _lib.use_cuda(x):
        # CPU oracle of the fp8 path: same routing, activations quantised per 1 x 128 block before each expert GEMM
        ids, w = route_ref(router_logits, top_k, renorm)
        w13f, w2f = w13.dequant(), w2.dequant()
        out = torch.zeros(T, H, dtype=torch.float32)
        for e in range(e0, e1):
            m = ids == e
            rows = m.any(-1).nonzero().flatten()
            if rows.numel():
                q, st = gemm_fp8.quantize_act_ref(x[rows])
                gu = F.linear(gemm_fp8._dequant_act(q, st), w13f[e - e0])
                h = (F.silu(gu[:, 0::2]) * gu[:, 1::2]).to(x.dtype)
                q2, st2 = gemm_fp8.quantize_act_ref(h)
                y = F.linear(gemm_fp8._dequant_act(q2, st2), w2f[e - e0])
                out[rows] += ((w * m)[rows].sum(-1, keepdim=True) * y).to(x.dtype).float()
        if add is not None:
            out += add.float()
        return out.to(x.dtype)
    if not _lib.use_cuda(x):
        ids, w = route_ref(router_logits, top_k, renorm)
        out = torch.zeros(T, H, dtype=torch.float32)
        for e in range(e0, e1):
            m = ids == e
            rows = m.any(-1).nonzero().flatten()
            if rows.numel():
                gu = F.linear(x[rows].float(), w13[e - e0].float())
                h = (F.silu(gu[:, 0::2]) * gu[:, 1::2]).to(x.dtype).float()
                out[rows] += (w * m)[rows].sum(-1, keepdim=True) * F.linear(h, w2[e - e0].float()).to(x.dtype).float()
        if add is not None:
            out += add.float()
        return out.to(x.dtype)
    L = _lib.kernels()
    s = ctypes.c_void_p(_lib.stream_ptr())
    br = choose_block_rows(T * top_k, E_local)
    ws = _workspace(x.device, T, top_k, E_local, H, I, br)
    _lib.check(L.mstar_moe_topk(_p(router_logits), T, E, top_k, 1 if renorm else 0, _p(ws.topk_ids), _p(ws.topk_w), s), "moe_topk")
    _lib.check(L.mstar_moe_align(_p(ws.topk_ids), _p(ws.topk_w), T * top_k, E, br, ws.capacity, e0, e1, _p(ws.sorted_pair),
                                 _p(ws.sorted_w), _p(ws.pos_of_pair), _p(ws.block_expert), _p(ws.num_blocks), s), "moe_align")
    if fp8:
        # token copies are gathered in expert order and quantised in one kernel; the SwiGLU output is quantised again
        # for the second expert GEMM
        x8, xs = gemm_fp8.quantize_act(x, src_row=ws.sorted_pair, src_div=top_k, rows=ws.capacity)
        _lib.check(L.mstar_moe_grouped_gemm_fp8(_p(x8), _p(xs), int(xs.stride(0)), _p(w13.data), _p(w13.scale),
                                                _p(ws.h_sorted), ws.capacity, 2 * I, H, E_local, br, _p(ws.block_expert),
                                                _p(ws.num_blocks), None, None, gemm.EPILOGUE_SWIGLU, I, s),
                   "moe_grouped_gemm_fp8 1")
        h8, hs = gemm_fp8.quantize_act(ws.h_sorted[:ws.capacity])
        _lib.check(L.mstar_moe_grouped_gemm_fp8(_p(h8), _p(hs), int(hs.stride(0)), _p(w2.data), _p(w2.scale),
                                                _p(ws.y_sorted), ws.capacity, H, I, E_local, br, _p(ws.block_expert),
                                                _p(ws.num_blocks), _p(ws.sorted_w), None, 0, H, s),
                   "moe_grouped_gemm_fp8 2")
        out = torch.empty(T, H, dtype=x.dtype, device=x.device)
        _lib.check(L.mstar_moe_unpermute(_p(ws.y_sorted), _p(ws.pos_of_pair), None, T, top_k, H, ctypes.c_longlong(H),
                                         _p(out), _p(add), s), "moe_unpermute")
        return out
    _lib.check(L.mstar_moe_permute(_p(x), _p(ws.sorted_pair), ws.capacity, H, top_k, _p(ws.x_sorted), None, s), "moe_permute")
    _lib.check(L.mstar_moe_grouped_gemm(_p(ws.x_sorted), _p(w13), _p(ws.h_sorted), ws.capacity, 2 * I, H, E_local, br,
                                        _p(ws.block_expert), _p(ws.num_blocks), None, None, gemm.EPILOGUE_SWIGLU, I, s),
               "moe_grouped_gemm 1")
    _lib.check(L.mstar_moe_grouped_gemm(_p(ws.h_sorted), _p(w2), _p(ws.y_sorted), ws.capacity, H, I, E_local, br,
                                        _p(ws.block_expert), _p(ws.num_blocks), _p(ws.sorted_w), None, 0, H, s),
               "moe_grouped_gemm 2")
    out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    _lib.check(L.mstar_moe_unpermute(_p(ws.y_sorted), _p(ws.pos_of_pair), None, T, top_k, H, ctypes.c_longlong(H), _p(out),
                                     _p(add), s), "moe_unpermute")
    return out
