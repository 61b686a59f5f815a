"""Expert parallelism over the symmetric heap: dispatch by peer stores, grouped GEMMs on the owner, combine as the
epilogue of the second GEMM (rows stored straight into the source rank's buffer), sum over k at the source.
Every rank of the group calls ``ep_moe`` with its own tokens (the same number of calls in the same order)."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib, gemm
from ..ops import moe as moe_ops


class _EpState:
    def __init__(self, heap, T_max: int, top_k: int, H: int, E_local: int, I: int):
        self.cap = T_max * top_k
        W = heap.world
        self.recv_x_off = heap.alloc_user(W * self.cap * H * 2)
        self.recv_meta_off = heap.alloc_user(W * self.cap * 16)
        self.recv_count_off = heap.alloc_user(64)
        self.combine_off = heap.alloc_user(self.cap * H * 2)
        d = heap.device
        n = W * self.cap
        self.send_counters = torch.zeros(8, dtype=torch.int32, device=d)
        self.ids_flat = torch.empty(n, dtype=torch.int32, device=d)
        self.w_flat = torch.empty(n, dtype=torch.float32, device=d)
        self.dst_flat = torch.zeros(n, dtype=torch.int64, device=d)
        self.topk_ids = torch.empty(T_max, top_k, dtype=torch.int32, device=d)
        self.topk_w = torch.empty(T_max, top_k, dtype=torch.float32, device=d)
        self.br = 16 if n // max(1, E_local) <= 16 * W else 64
        self.capacity = (n + E_local * (self.br - 1) + self.br - 1) // self.br * self.br
        self.sorted_pair = torch.empty(self.capacity, dtype=torch.int32, device=d)
        self.sorted_w = torch.empty(self.capacity, dtype=torch.float32, device=d)
        self.pos_unused = torch.empty(n, dtype=torch.int32, device=d)
        self.block_expert = torch.zeros(self.capacity // self.br, dtype=torch.int32, device=d)
        self.num_blocks = torch.zeros(1, dtype=torch.int32, device=d)
        self.row_dst = torch.zeros(self.capacity, dtype=torch.int64, device=d)
        self.x_sorted = torch.zeros(self.capacity, H, dtype=torch.bfloat16, device=d)
        self.h_sorted = torch.empty(self.capacity, I, dtype=torch.bfloat16, device=d)
        self.identity_pos = torch.arange(self.cap, dtype=torch.int32, device=d)
        self.recv_x = heap.local_view(self.recv_x_off, (n, H), torch.bfloat16)
        self.combine = heap.local_view(self.combine_off, (self.cap, H), torch.bfloat16)


def _p(t):
    return ctypes.c_void_p(_lib.ptr(t))


def ep_moe(block, h: torch.Tensor, logits: torch.Tensor, add: torch.Tensor | None = None, T_max: int = 512):
    """``block``: SparseMoeBlock in EP mode (holds w13 / w2 of the local experts). h [T,H] bf16, logits [T,E]."""
    heap = block.ep.symm
    T, H = h.shape
    k, El, I = block.top_k, block.E_local, block.I_local
    st = getattr(block, "_ep_state", None)
    if st is None:
        st = _EpState(heap, max(T_max, T), k, H, El, I)
        # one state (and one set of heap buffers) is shared by all layers of a model: the calls are serialised
        block._ep_state = st
    L = _lib.kernels()
    s = ctypes.c_void_p(_lib.stream_ptr())
    bufs, flags = heap.tables()
    W, R = heap.world, heap.rank
    ids, w = st.topk_ids[:T], st.topk_w[:T]
    _lib.check(L.mstar_moe_topk(_p(logits), T, block.E, k, 1 if block.cfg.norm_topk_prob else 0, _p(ids), _p(w), s), "moe_topk")
    heap.barrier()      # the previous call's combine rows have been consumed everywhere before buffers are reused
    _lib.check(L.mstar_ep_dispatch(bufs, flags, W, R, _p(h), _p(ids), _p(w), T * k, k, H, El, st.cap,
                                   ctypes.c_longlong(st.recv_x_off), ctypes.c_longlong(st.recv_meta_off),
                                   ctypes.c_longlong(st.recv_count_off), _p(st.send_counters), s), "ep_dispatch")
    heap.barrier()      # all rows and counts have landed
    _lib.check(L.mstar_ep_prepare(bufs, flags, W, R, st.cap, H, k, ctypes.c_longlong(st.recv_meta_off),
                                  ctypes.c_longlong(st.recv_count_off), ctypes.c_longlong(st.combine_off),
                                  _p(st.ids_flat), _p(st.w_flat), _p(st.dst_flat), s), "ep_prepare")
    n = W * st.cap
    _lib.check(L.mstar_moe_align(_p(st.ids_flat), _p(st.w_flat), n, El, st.br, st.capacity, 0, El, _p(st.sorted_pair),
                                 _p(st.sorted_w), _p(st.pos_unused), _p(st.block_expert), _p(st.num_blocks), s), "moe_align")
    _lib.check(L.mstar_moe_permute(_p(st.recv_x), _p(st.sorted_pair), st.capacity, H, 1, _p(st.x_sorted), None, s), "moe_permute")
    _lib.check(L.mstar_gather_ptrs(_p(st.dst_flat), _p(st.sorted_pair), st.capacity, _p(st.row_dst), s), "gather_ptrs")
    _lib.check(L.mstar_moe_grouped_gemm(_p(st.x_sorted), _p(block.w13), _p(st.h_sorted), st.capacity, 2 * I, H, El, st.br,
                                        _p(st.block_expert), _p(st.num_blocks), None, None, gemm.EPILOGUE_SWIGLU, I, s), "ep gemm 1")
    # second GEMM: routing weight and the combine store (to the source rank's buffer, over NVLink) in the epilogue
    _lib.check(L.mstar_moe_grouped_gemm(_p(st.h_sorted), _p(block.w2), None, st.capacity, H, I, El, st.br,
                                        _p(st.block_expert), _p(st.num_blocks), _p(st.sorted_w), _p(st.row_dst), 0, H, s), "ep gemm 2")
    heap.barrier()      # every owner has stored its rows into this rank's combine buffer
    out = torch.empty(T, H, dtype=h.dtype, device=h.device)
    _lib.check(L.mstar_moe_unpermute(_p(st.combine), _p(st.identity_pos), None, T, k, H, ctypes.c_longlong(H), _p(out),
                                     _p(add), s), "moe_unpermute")
    return out
