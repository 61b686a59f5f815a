"""Symmetric heap: one buffer per rank of a group, mapped into every rank's address space, plus flag words for
device-side signalling. The allocation and the handle exchange use ``torch.distributed._symmetric_memory``
(bootstrap plumbing over the NCCL/gloo store); everything that moves data afterwards is this library's own
kernels (``csrc/comm.cu``, the fused GEMM epilogue) issuing plain peer loads / stores over NVLink.

Layout of every rank's heap:
    [ reduce slots: 2 x slot_bytes ][ user region: user_bytes ][ flags: n_channels x 8 x u32 ]
Local (non-shared) state words hold the epochs of the channel sets.

Reference counterparts: NCCL process groups through torch.distributed (mstar/distributed/communication.py:
214-263) — collectives there are separate library kernels between the GEMMs; here the heap lets a kernel read or
write a peer's memory while it computes.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib

MAX_RANKS = 8
N_CHANNELS = 4096
# channel map
CH_ALLREDUCE = 0          # [0, 512): all-reduce CTAs (two rounds of up to 256)
CH_BARRIER = 512
CH_A2A = 513              # [513, 521)
CH_CFG = 528
CH_GEMM_AR = 544          # [544, 1024): fused GEMM + all-reduce tiles
CH_NVLS_AR = 1024         # [1024, 1280): NVLS all-reduce CTAs (two rounds of up to 128)
CH_RRN = 1280             # [1280, 2305): reduce + residual + norm consumers (1 + up to 1024 blocks of the two-shot form)
CH_AG = 2432              # [2432, 2560): column all-gather CTAs
CH_AR_INPLACE = 2560      # [2560, 2816): in-place all-reduce CTAs (two rounds of up to 128)
CH_GEMM_TILES = 2816      # [2816, 2944): row groups of the GEMM with the all-reduce inside (two rounds of up to 64)
# local state words (pairs of [epoch, arrive]) by user
ST_AR, ST_BARRIER, ST_A2A, ST_CFG, ST_GEMM_AR, ST_NVLS_AR, ST_RRN, ST_AG, ST_AR_INPLACE = range(9)


class SymmRegion:
    """An additional symmetric allocation of a group (same size on every rank, every rank's copy mapped into every
    rank, bound to one NVLS multicast object when the box has them). Models carve their tensor-parallel buffers out
    of regions: partial-sum slots of row-parallel projections, vocabulary shards, gathered logits."""

    def __init__(self, heap: "SymmetricHeap", nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem
        self.heap = heap
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=heap.device)
        self.buf.zero_()
        handle = symm_mem.rendezvous(self.buf, group=heap.group_name)
        self.handle = handle
        self.ptrs = [int(p) for p in handle.buffer_ptrs]
        self.mc_ptr = int(getattr(handle, "multicast_ptr", 0) or 0) if heap.use_multicast else 0
        self.table = (ctypes.c_void_p * MAX_RANKS)(*([ctypes.c_void_p(p) for p in self.ptrs] + [None] * (MAX_RANKS - heap.world)))
        self._cursor = 0
        torch.cuda.synchronize(heap.device)
        dist.barrier(group=heap.group)

    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError("symmetric region exhausted")
        self._cursor = off + nbytes
        return off

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buf[offset:offset + nbytes].view(dtype).view(*shape)


class SymmetricHeap:
    def __init__(self, group: "dist.ProcessGroup", ranks: list[int], rank: int, device,
                 slot_bytes: int = 32 << 20, user_bytes: int = 64 << 20):
        import torch.distributed._symmetric_memory as symm_mem
        self.device = torch.device(device)
        self.world = len(ranks)
        self.rank = ranks.index(rank)
        self.slot_bytes = slot_bytes
        self.user_bytes = user_bytes
        self.flag_bytes = N_CHANNELS * MAX_RANKS * 4
        total = 2 * slot_bytes + user_bytes + self.flag_bytes
        gname = group.group_name if hasattr(group, "group_name") else group
        self.group_name = gname
        self.group = group
        # NVLS: on when the rendezvous hands back a multicast address (MSTAR_NVLS=0 forces the plain peer paths)
        import os
        self.use_multicast = os.environ.get("MSTAR_NVLS", "1") != "0"
        try:
            symm_mem.enable_symm_mem_for_group(gname)      # needed on older torch, a no-op warning on newer
        except Exception:
            pass
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group=gname)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world
        self.base_ptrs = ptrs
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) if self.use_multicast else 0
        self.mc_flags = (self.mc_ptr + 2 * slot_bytes + user_bytes) if self.mc_ptr else 0
        self._bufs = (ctypes.c_void_p * MAX_RANKS)(*([ctypes.c_void_p(p) for p in ptrs] + [None] * (MAX_RANKS - self.world)))
        fl = [p + 2 * slot_bytes + user_bytes for p in ptrs]
        self._flags = (ctypes.c_void_p * MAX_RANKS)(*([ctypes.c_void_p(p) for p in fl] + [None] * (MAX_RANKS - self.world)))
        self.user_offset = 2 * slot_bytes
        # local state: [epoch, arrive] pairs per channel set
        self.state = torch.zeros(64, dtype=torch.int32, device=self.device)
        self._user_cursor = 0
        # the fused GEMM + all-reduce epilogue has its own pair of slots (its epochs are independent of the
        # stand-alone all-reduce, so the two must never share a slot)
        self.gemm_slot_bytes = 8 << 20
        goff = self.alloc_user(2 * self.gemm_slot_bytes)
        self._gemm_bufs = (ctypes.c_void_p * MAX_RANKS)(
            *([ctypes.c_void_p(p + goff) for p in ptrs] + [None] * (MAX_RANKS - self.world)))
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # ---- user region carving (same order on every rank => symmetric offsets) ----
    def alloc_user(self, nbytes: int, align: int = 256) -> int:
        off = (self._user_cursor + align - 1) // align * align
        if off + nbytes > self.user_bytes:
            raise MemoryError("symmetric heap user region exhausted")
        self._user_cursor = off + nbytes
        return self.user_offset + off

    def local_view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buf[offset:offset + nbytes].view(dtype).view(*shape)

    def _state_ptr(self, idx: int) -> ctypes.c_void_p:
        return ctypes.c_void_p(self.state.data_ptr() + idx * 8)

    # ---- collectives ----
    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                   mode: int = 0) -> torch.Tensor:
        """Sum of ``x`` (bf16, contiguous, numel % 8 == 0) over the group; every rank gets the identical result."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        n = x.numel()
        # messages larger than a heap slot go in slot-sized pieces (two-shot keeps partials and results in one slot)
        # (one-shot: one region per rank in the slot; two-shot: received shares + margin | gathered result)
        one_shot = mode == 1 or (mode == 0 and self.world <= 2)
        if one_shot:
            piece = (self.slot_bytes // (2 * self.world)) // 8 * 8
        else:
            piece = ((self.slot_bytes // 2 - (64 << 10)) // 2) // 8 * 8
        xf, of = x.view(-1), out.view(-1)
        rf = residual.view(-1) if residual is not None else None
        for a in range(0, n, piece):
            b = min(n, a + piece)
            rc = _lib.kernels().mstar_allreduce(
                self._bufs, self._flags, self.world, self.rank, ctypes.c_void_p(xf[a:b].data_ptr()),
                ctypes.c_void_p(of[a:b].data_ptr()), ctypes.c_void_p(_lib.ptr(rf[a:b]) if rf is not None else 0),
                ctypes.c_longlong(b - a), ctypes.c_longlong(self.slot_bytes), self._state_ptr(ST_AR), CH_ALLREDUCE, 128,
                int(mode), ctypes.c_void_p(_lib.stream_ptr()))
            if rc < 0:
                _lib.check(rc, "mstar_allreduce")
        return out

    def barrier(self) -> None:
        rc = _lib.kernels().mstar_peer_barrier(self._bufs, self._flags, self.world, self.rank, self._state_ptr(ST_BARRIER),
                                               CH_BARRIER, ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_peer_barrier")

    def a2a_heads(self, src: torch.Tensor, dst_offset: int, forward: bool, H: int, D: int, seq_off: list[int]) -> None:
        """Ulysses exchange by peer stores into the tensor at ``dst_offset`` of every rank's heap; returns after
        the peers' stores into this rank's tensor are visible to later kernels of the stream."""
        assert src.dtype == torch.bfloat16 and src.is_contiguous()
        so = (ctypes.c_int * (MAX_RANKS + 1))(*(list(seq_off) + [seq_off[-1]] * (MAX_RANKS + 1 - len(seq_off))))
        rc = _lib.kernels().mstar_a2a_heads(self._bufs, self._flags, self.world, self.rank,
                                            ctypes.c_void_p(src.data_ptr()), ctypes.c_longlong(dst_offset),
                                            1 if forward else 0, int(H), int(D), so, self._state_ptr(2), CH_A2A,
                                            ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_a2a_heads")

    def rope_scatter(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                     axis_of_freq: torch.Tensor | None, q_norm_w, k_norm_w, norm_eps: float, Hq: int, Hkv: int, D: int,
                     q_off: int, k_off: int, v_off: int, seq_off: list[int], interleaved: bool = False) -> None:
        """QK-norm + RoPE of this rank's projection rows with the Ulysses head scatter as the store: every head goes
        straight into the q / k / v tensor (at ``q_off`` / ``k_off`` / ``v_off`` of the heap) of the rank that attends
        with it. Returns after the peers' stores into this rank's tensors are visible to later kernels."""
        assert qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.stride(1) == 1
        pos = positions if positions.dim() == 2 else positions[None]
        assert pos.dtype == torch.int32 and pos.stride(1) == 1
        so = (ctypes.c_int * (MAX_RANKS + 1))(*(list(seq_off) + [seq_off[-1]] * (MAX_RANKS + 1 - len(seq_off))))
        rc = _lib.kernels().mstar_rope_scatter(
            self._bufs, self._flags, self.world, self.rank, ctypes.c_void_p(qkv.data_ptr()),
            ctypes.c_longlong(qkv.stride(0)), ctypes.c_void_p(pos.data_ptr()), ctypes.c_longlong(pos.stride(0)),
            ctypes.c_void_p(inv_freq.data_ptr()), ctypes.c_void_p(_lib.ptr(axis_of_freq)),
            ctypes.c_void_p(_lib.ptr(q_norm_w)), ctypes.c_void_p(_lib.ptr(k_norm_w)), ctypes.c_longlong(q_off),
            ctypes.c_longlong(k_off), ctypes.c_longlong(v_off), int(qkv.shape[0]), int(Hq), int(Hkv), int(D),
            1 if interleaved else 0, ctypes.c_float(norm_eps), so, self._state_ptr(2), CH_A2A,
            ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_rope_scatter")
        _lib._counters.bump()

    def signal(self, dst_rank: int, channel: int = CH_CFG, state_idx: int = 3, bump: bool = True) -> None:
        rc = _lib.kernels().mstar_peer_signal(self._bufs, self._flags, self.world, self.rank,
                                              self._state_ptr(state_idx), int(channel), int(dst_rank),
                                              1 if bump else 0, ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_peer_signal")

    def cfg_combine(self, v_offset: int, cond_rank: int, uncond_rank: int, img_rank: int, x: torch.Tensor,
                    dt: float, s_text: float, s_img: float = 1.0, renorm: bool = False, renorm_min: float = 0.0,
                    wait_peers: bool = True):
        """Guidance combine on this rank, reading the branch velocities (fp32 [rows, cols] at ``v_offset`` of the
        branch ranks' heaps) over NVLink. Returns (x_next, v)."""
        rows, cols = x.shape
        x = x.float().contiguous()
        x_next, v = torch.empty_like(x), torch.empty_like(x)
        rc = _lib.kernels().mstar_cfg_combine_peer(
            self._bufs, self._flags, self.world, self.rank, ctypes.c_longlong(v_offset), int(cond_rank),
            int(uncond_rank), int(img_rank), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x_next.data_ptr()),
            ctypes.c_void_p(v.data_ptr()), int(rows), int(cols), ctypes.c_float(s_text), ctypes.c_float(s_img),
            ctypes.c_float(dt), 1 if renorm else 0, ctypes.c_float(renorm_min), self._state_ptr(3), CH_CFG,
            1 if wait_peers else 0, ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_cfg_combine_peer")
        return x_next, v

    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                          residual: torch.Tensor | None = None) -> torch.Tensor:
        """Row-parallel projection: ``sum_over_ranks(x_r @ w_r.T) (+bias) (+residual)`` in ONE kernel per rank —
        the tcgen05 GEMM publishes each output tile in the heap and sums the peers' tiles in its epilogue.
        Decode layout only (at most 128 rows); larger inputs take GEMM + stand-alone all-reduce."""
        from ..ops import gemm
        M = x.numel() // x.shape[-1]
        N = w.shape[0]
        if M > 128 or N % 8 or self.world * M * N * 2 > self.gemm_slot_bytes:
            y = gemm.linear(x, w, bias=bias if self.rank == 0 else None)
            return self.all_reduce(y.contiguous(), residual=residual)
        rc = _lib.kernels().mstar_gemm_arm_allreduce(self._gemm_bufs, self._flags, self.world, self.rank,
                                                     ctypes.c_longlong(self.gemm_slot_bytes), self._state_ptr(4),
                                                     CH_GEMM_AR)
        _lib.check(rc, "mstar_gemm_arm_allreduce")
        return gemm.linear(x, w, bias=bias if self.rank == 0 else None, residual=residual)

    # ---- NVLS paths (multicast loads / stores through the switch, plain peer accesses as the fallback) ----
    def new_region(self, nbytes: int) -> SymmRegion:
        """Collective: every rank of the group calls it with the same size, in the same order."""
        return SymmRegion(self, nbytes)

    def _mc(self, region: SymmRegion | None):
        data = region.mc_ptr if region is not None else self.mc_ptr
        return ctypes.c_void_p(data or None), ctypes.c_void_p(self.mc_flags or None)

    def all_reduce_nvls(self, x: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                        mode: int = 0) -> torch.Tensor:
        """All-reduce whose additions happen inside the NVSwitch (``multimem.ld_reduce``); two-shot form for large
        messages multicast-stores each rank's share of the sum to all ranks. Staged through the heap's reduce slots."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        n = x.numel()
        piece = (self.slot_bytes // 4) // 8 * 8            # a slot holds [input | gathered result] of one piece
        xf, of = x.view(-1), out.view(-1)
        rf = residual.view(-1) if residual is not None else None
        mc_data, mc_flags = self._mc(None)
        for a in range(0, n, piece):
            b = min(n, a + piece)
            rc = _lib.kernels().mstar_allreduce_nvls(
                self._bufs, self._flags, self.world, self.rank, mc_data, mc_flags,
                ctypes.c_void_p(xf[a:b].data_ptr()), ctypes.c_void_p(of[a:b].data_ptr()),
                ctypes.c_void_p(_lib.ptr(rf[a:b]) if rf is not None else 0), ctypes.c_longlong(b - a),
                ctypes.c_longlong(0), ctypes.c_longlong(self.slot_bytes), self._state_ptr(ST_NVLS_AR), CH_NVLS_AR, 128,
                int(mode), ctypes.c_void_p(_lib.stream_ptr()))
            if rc < 0:
                _lib.check(rc, "mstar_allreduce_nvls")
            _lib._counters.bump()
        return out

    def all_reduce_inplace(self, region: SymmRegion, off: int, n: int) -> None:
        """Sum, over the group, of the bf16 tensor of ``n`` elements at byte offset ``off`` of ``region``; the result
        replaces it on every rank. For producers that write their partial straight into the region (a row-parallel
        GEMM with ``out=region.view(...)``): nothing is staged or copied, the additions happen in the switch."""
        mc_data, mc_flags = self._mc(region)
        rc = _lib.kernels().mstar_allreduce_inplace(
            region.table, self._flags, self.world, self.rank, mc_data, mc_flags, ctypes.c_longlong(off),
            ctypes.c_longlong(n), self._state_ptr(ST_AR_INPLACE), CH_AR_INPLACE, 128,
            ctypes.c_void_p(_lib.stream_ptr()))
        if rc < 0:
            _lib.check(rc, "mstar_allreduce_inplace")
        _lib._counters.bump()

    def scratch(self, nbytes: int) -> tuple[SymmRegion, int]:
        """A symmetric scratch area of at least ``nbytes`` (region, byte offset). Collective when it has to grow:
        every rank asks for the same sizes in the same order. A result kept there must be consumed before the next
        call that uses the scratch (stream order is enough: a kernel that reduces into it returns only after every
        peer has finished reading and writing this rank's copy)."""
        reg = getattr(self, "_scratch", None)
        if reg is None or reg.nbytes < nbytes:
            self._scratch = reg = self.new_region(max(nbytes, 64 << 20))
            self._scratch_off = reg.alloc(reg.nbytes - 4096)
        return reg, self._scratch_off

    def linear_all_reduce_tiles(self, x: torch.Tensor, w: torch.Tensor, region: SymmRegion, off: int,
                                bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                                n_comm: int = 0, group_p: int = 0) -> torch.Tensor:
        """Row-parallel projection at large M with the all-reduce inside the GEMM kernel: ``sum_ranks x_r @ w_r.T``
        (+ bias, + residual: pass them on one rank only) lands, summed, at byte offset ``off`` of ``region`` on every
        rank; the returned tensor is that view. Communication CTAs of the same launch reduce finished row groups
        over peer memory while the remaining tiles are still being multiplied. The region must have room for C and,
        behind it, a staging area of about the same size (``2 * M * N * 2`` bytes from ``off`` are always enough)."""
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
        M, K = x.shape
        N = w.shape[0]
        if not hasattr(self, "_tile_ctrs"):
            self._tile_ctrs = torch.zeros(256, dtype=torch.int32, device=self.device)
        _, mc_flags = self._mc(region)
        c_bytes = (M * N * 2 + 255) // 256 * 256
        stage_off = off + c_bytes                           # the peers' pushes land behind C
        stage_bytes = region.nbytes - stage_off
        rc = _lib.kernels().mstar_gemm_bf16_allreduce_tiles(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), int(M), int(N), int(K), int(x.stride(0)),
            int(w.stride(0)), ctypes.c_void_p(_lib.ptr(bias) if bias is not None else 0),
            ctypes.c_void_p(_lib.ptr(residual) if residual is not None else 0),
            int(residual.stride(0)) if residual is not None else 0, region.table, self._flags, self.world, self.rank,
            mc_flags, ctypes.c_longlong(off), ctypes.c_longlong(stage_off), ctypes.c_longlong(stage_bytes),
            ctypes.c_void_p(self._tile_ctrs.data_ptr()), CH_GEMM_TILES, int(n_comm), int(group_p),
            ctypes.c_void_p(_lib.stream_ptr()))
        if rc < 0:
            _lib.check(rc, "mstar_gemm_bf16_allreduce_tiles")
        _lib._counters.bump()
        return region.view(off, (M, N), torch.bfloat16)

    def row_share(self, M: int) -> tuple[int, int]:
        """Rows [a, b) of an M-row activation that this rank owns in the two-shot (row-cut) forms."""
        per = (M + self.world - 1) // self.world
        a = min(M, self.rank * per)
        return a, min(M, a + per)

    def reduce_residual_norm(self, region: SymmRegion, slot_off: int, M: int, N: int, gamma: torch.Tensor | None,
                             eps: float, residual: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                             want_residual: bool = True, h_off: int | None = None):
        """Consumer of a row-parallel projection whose PARTIAL output every rank wrote at ``slot_off`` of its copy of
        ``region``: sum over ranks (in the switch) + bias + residual -> new residual; RMSNorm -> out. Returns
        (normalised [M, N], new residual or None).

        With ``h_off`` (two-shot form, for large M): this rank reduces and normalises only its row share
        (``row_share``), multicast-stores the rows into the [M, N] buffer at ``h_off`` of every rank's region copy,
        and waits until the peers' rows are in its own copy. ``residual`` and the returned residual then hold this
        rank's rows only (the residual stream stays cut by rows); the returned ``out`` is the local view at
        ``h_off``."""
        two_shot = h_off is not None
        a, b = self.row_share(M) if two_shot else (0, M)
        out = region.view(h_off, (M, N), torch.bfloat16) if two_shot else \
            torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        res_out = torch.empty((b - a, N), dtype=torch.bfloat16, device=self.device) if want_residual else None
        mc_data, mc_flags = self._mc(region)
        rc = _lib.kernels().mstar_reduce_residual_norm(
            region.table, self._flags, self.world, self.rank, mc_data, mc_flags, ctypes.c_longlong(slot_off), int(M),
            int(N), ctypes.c_void_p(_lib.ptr(residual)), ctypes.c_void_p(_lib.ptr(res_out)),
            ctypes.c_void_p(_lib.ptr(gamma)), ctypes.c_void_p(_lib.ptr(bias)),
            ctypes.c_void_p(0 if two_shot else out.data_ptr()), ctypes.c_float(eps), 1 if two_shot else 0, int(a),
            int(b), ctypes.c_longlong(h_off or 0), self._state_ptr(ST_RRN), CH_RRN, ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_reduce_residual_norm")
        return out, res_out

    def allgather_cols(self, region: SymmRegion, shard_off: int, full_off: int, M: int, Ns: int) -> None:
        """Every rank's [M, Ns] shard (at ``shard_off`` of its region copy) lands at columns [rank * Ns, ...) of the
        [M, world * Ns] matrix at ``full_off`` on every rank."""
        mc_data, mc_flags = self._mc(region)
        rc = _lib.kernels().mstar_allgather_cols(region.table, self._flags, self.world, self.rank, mc_data, mc_flags,
                                                 ctypes.c_longlong(shard_off), ctypes.c_longlong(full_off), int(M),
                                                 int(Ns), self._state_ptr(ST_AG), CH_AG, 128,
                                                 ctypes.c_void_p(_lib.stream_ptr()))
        if rc < 0:
            _lib.check(rc, "mstar_allgather_cols")
        _lib._counters.bump()

    def embed_gather(self, region: SymmRegion, table_off: int, rows_per_rank: int, H: int, ids: torch.Tensor,
                     vocab: int) -> torch.Tensor:
        """Rows of a vocabulary-parallel embedding table, each loaded from the shard of the rank that owns it."""
        flat = ids.reshape(-1).contiguous()
        out = torch.empty((flat.numel(), H), dtype=torch.bfloat16, device=self.device)
        rc = _lib.kernels().mstar_embed_gather_p2p(region.table, self.world, self.rank, ctypes.c_longlong(table_off),
                                                   int(rows_per_rank), int(H), ctypes.c_void_p(flat.data_ptr()),
                                                   ctypes.c_void_p(out.data_ptr()), int(flat.numel()), int(vocab),
                                                   ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_embed_gather_p2p")
        return out

    # ---- table for fused kernels ----
    def tables(self):
        return self._bufs, self._flags


def attach_symmetric_heap(group, device, **kw) -> SymmetricHeap | None:
    """Create the heap for a ``CommGroup`` and hang it on ``group.symm``. Returns None (and leaves the NCCL path
    in place) for trivial groups or CPU ranks."""
    if group.size <= 1 or not torch.cuda.is_available():
        return None
    heap = SymmetricHeap(group.group, group.ranks, group.global_rank, device, **kw)
    group.symm = heap
    return heap
