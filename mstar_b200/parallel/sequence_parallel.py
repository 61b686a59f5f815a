"""Ulysses sequence parallelism: the residual stream is sharded along the sequence ([S/P, H] per rank) for all
pointwise ops and MLPs; around attention the layout flips to head-sharded over the FULL sequence.

GPU path: the exchange is peer stores over the symmetric heap (``SymmetricHeap.a2a_heads``: every rank writes its
rows of each head group straight into the owner's attention input buffer, and the attention output rows straight
back into the owners' sequence shards); it is a fixed sequence of kernels, so it captures into CUDA graphs (the
reference swaps its send/recv all-to-all for all-gathers under capture). CPU ranks (gloo) and ranks without a
heap use ``all_gather`` + slicing, which has the same result.

Reference counterparts: ``sp_seq_split`` / ``scatter_sequence`` / ``gather_sequence`` / ``ulysses_attention`` /
``_ulysses_attention_via_all_gather`` / ``sp_head_slice`` / ``sp_head_gather``
(mstar/model/components/distributed/sequence_parallel.py:31-176).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .comm import CommGroup


def sp_seq_split(S: int, P: int) -> list[int]:
    """Row offsets (P + 1) of the sequence shards; the first S % P ranks get one extra row."""
    base, extra = divmod(S, P)
    off = [0]
    for r in range(P):
        off.append(off[-1] + base + (1 if r < extra else 0))
    return off


def scatter_sequence(x: torch.Tensor, sp: CommGroup, dim: int = 0) -> torch.Tensor:
    if sp.size == 1:
        return x
    off = sp_seq_split(x.shape[dim], sp.size)
    return x.narrow(dim, off[sp.rank], off[sp.rank + 1] - off[sp.rank]).contiguous()


def gather_sequence(x: torch.Tensor, sp: CommGroup, S: int, dim: int = 0) -> torch.Tensor:
    """All ranks get the full sequence (shards padded to the largest for the collective)."""
    if sp.size == 1:
        return x
    off = sp_seq_split(S, sp.size)
    mx = max(off[r + 1] - off[r] for r in range(sp.size))
    xt = x.transpose(0, dim) if dim != 0 else x
    pad = torch.zeros((mx, *xt.shape[1:]), dtype=x.dtype, device=x.device)
    pad[:xt.shape[0]] = xt
    parts = [torch.empty_like(pad) for _ in range(sp.size)]
    dist.all_gather(parts, pad.contiguous(), group=sp.group)
    full = torch.cat([p[:off[r + 1] - off[r]] for r, p in enumerate(parts)], dim=0)
    return full.transpose(0, dim) if dim != 0 else full


def sp_head_slice(x: torch.Tensor, sp: CommGroup, head_dim_index: int = 1) -> torch.Tensor:
    """This rank's head group of a replicated [*, H, D] tensor (text-prefix K/V that every rank holds)."""
    if sp.size == 1:
        return x
    Hp = x.shape[head_dim_index] // sp.size
    return x.narrow(head_dim_index, sp.rank * Hp, Hp).contiguous()


def sp_head_gather(x: torch.Tensor, sp: CommGroup, head_dim_index: int = 1) -> torch.Tensor:
    if sp.size == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(sp.size)]
    dist.all_gather(parts, x.contiguous(), group=sp.group)
    return torch.cat(parts, dim=head_dim_index)


class UlyssesExchange:
    """Buffers and offsets of one (sequence length, head counts) configuration."""

    def __init__(self, sp: CommGroup, S: int, Hq: int, Hkv: int, D: int, dtype=torch.bfloat16):
        self.sp, self.S, self.Hq, self.Hkv, self.D = sp, S, Hq, Hkv, D
        self.off = sp_seq_split(S, sp.size)
        self.heap = getattr(sp, "symm", None)
        P = sp.size
        if self.heap is not None:
            e = torch.empty((), dtype=dtype).element_size()
            self.q_off = self.heap.alloc_user(S * (Hq // P) * D * e)
            self.k_off = self.heap.alloc_user(S * (Hkv // P) * D * e)
            self.v_off = self.heap.alloc_user(S * (Hkv // P) * D * e)
            mx = max(self.off[r + 1] - self.off[r] for r in range(P))
            self.o_off = self.heap.alloc_user(mx * Hq * D * e)
            self.dtype = dtype

    def to_heads(self, q, k, v):
        """[S_loc, H, D] x3 -> [S, H/P, D] x3 (this rank's head group over the full sequence)."""
        sp, P = self.sp, self.sp.size
        if P == 1:
            return q, k, v
        if self.heap is not None and q.is_cuda:
            h = self.heap
            h.a2a_heads(q.contiguous(), self.q_off, True, self.Hq, self.D, self.off)
            h.a2a_heads(k.contiguous(), self.k_off, True, self.Hkv, self.D, self.off)
            h.a2a_heads(v.contiguous(), self.v_off, True, self.Hkv, self.D, self.off)
            return (h.local_view(self.q_off, (self.S, self.Hq // P, self.D), self.dtype),
                    h.local_view(self.k_off, (self.S, self.Hkv // P, self.D), self.dtype),
                    h.local_view(self.v_off, (self.S, self.Hkv // P, self.D), self.dtype))
        outs = []
        for t in (q, k, v):
            full = gather_sequence(t, sp, self.S)
            outs.append(sp_head_slice(full, sp, 1))
        return tuple(outs)

    def can_fuse_rope(self, qkv: torch.Tensor, rot_dim: int) -> bool:
        """The fused QK-norm + RoPE + head scatter kernel applies: peer heap, bf16 on a GPU, full rotary, head width
        64 or 128 (``MSTAR_ROPE_SCATTER=0`` keeps the separate RoPE kernel and exchange kernels)."""
        import os
        return (self.sp.size > 1 and self.heap is not None and qkv.is_cuda and qkv.dtype == torch.bfloat16
                and rot_dim == self.D and self.D in (64, 128) and os.environ.get("MSTAR_ROPE_SCATTER", "1") != "0")

    def rope_to_heads(self, qkv, positions, inv_freq, axis_of_freq, q_norm_w, k_norm_w, norm_eps, interleaved=False):
        """[S_loc, (Hq + 2 Hkv) * D] projection rows -> normalised, rotated q / k / v of this rank's head group over
        the full sequence ([S, H/P, D] x3), in ONE kernel whose stores are the exchange."""
        P, h = self.sp.size, self.heap
        h.rope_scatter(qkv, positions, inv_freq, axis_of_freq, q_norm_w, k_norm_w, norm_eps, self.Hq, self.Hkv, self.D,
                       self.q_off, self.k_off, self.v_off, self.off, interleaved)
        return (h.local_view(self.q_off, (self.S, self.Hq // P, self.D), self.dtype),
                h.local_view(self.k_off, (self.S, self.Hkv // P, self.D), self.dtype),
                h.local_view(self.v_off, (self.S, self.Hkv // P, self.D), self.dtype))

    def to_sequence(self, o):
        """[S, Hq/P, D] -> [S_loc, Hq, D]."""
        sp, P = self.sp, self.sp.size
        if P == 1:
            return o
        n_loc = self.off[sp.rank + 1] - self.off[sp.rank]
        if self.heap is not None and o.is_cuda:
            self.heap.a2a_heads(o.contiguous(), self.o_off, False, self.Hq, self.D, self.off)
            return self.heap.local_view(self.o_off, (n_loc, self.Hq, self.D), self.dtype)
        full = sp_head_gather(o, sp, 1)
        return full[self.off[sp.rank]:self.off[sp.rank + 1]].contiguous()
