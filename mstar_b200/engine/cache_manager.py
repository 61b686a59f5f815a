"""Batch planning over the paged KV pool.

``BatchedCacheManager.plan`` turns a list of (request, label, new-token count) into ONE packed int32 buffer —
q_indptr, kv_lens, page tables, rope positions, per-token cache slots, logit rows, sampler slots — staged in
pinned host memory and copied to a fixed device buffer with a single async H2D copy. Kernels read the plan from
the device buffer, so a captured CUDA graph is replayed after the host has only rewritten that buffer; decode
steps can also advance the plan on the device (``advance_on_device``) with no host work at all.

Reference counterparts: ``build_paged_indptrs`` (mstar/engine/cache_manager.py:36-62), ``BatchedCacheManager``
(:149-674: plan_rope :346-436, plan_rope_batched_cfg :439-480, advance_seq_lens :587-631, snapshot_all :634-665),
``FlashInferCacheManager.plan_attention[_batched_cfg]`` (:685-1020) whose host-side FlashInfer plan is replaced by
the device-read plan, ``DenseGenCacheManager`` (:1266-1488; dense attention over [prefix | fresh] is the same
kernel in dense mode here).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..ops import attention as attn_ops
from ..ops import elementwise as ew_ops
from ..utils import io_counters
from .kv_store import KVCacheConfig, PagedAllocationManager


@dataclass
class BatchContext:
    """Everything a model forward needs to know about the batch it runs on."""
    plan: attn_ops.AttnPlan
    positions: torch.Tensor            # int32 [n_axes, T]
    token_req: torch.Tensor            # int32 [T] batch entry of each token (-1: padding, no cache write)
    cache_pos: torch.Tensor            # int32 [T] position inside the entry's sequence (cache slot)
    logit_rows: torch.Tensor           # int64 [B] row of each entry's last token
    row_slot: torch.Tensor             # int32 [B] sampler slot of each entry
    kv_layers: list[torch.Tensor]
    num_tokens: int
    batch: int
    request_ids: list[str] = field(default_factory=list)
    labels: list[str] = field(default_factory=list)
    q_lens: list[int] = field(default_factory=list)
    write_cache: bool = True
    layer_idx: int = 0

    def kv(self, layer: int) -> torch.Tensor:
        return self.kv_layers[layer]


class _PlanBuffers:
    """One packed int32 device buffer (fixed address, so captured graphs can read it) and ``n_host`` pinned host
    staging buffers used in turn: the CPU may fill staging buffer N+1 while the copy of buffer N is still queued.
    Before a staging buffer is reused, the event recorded after its last upload is waited for."""

    def __init__(self, device, max_batch: int, max_tokens: int, max_pages: int, n_axes: int, n_host: int = 2):
        self.device = torch.device(device)
        self.max_batch, self.max_tokens, self.max_pages, self.n_axes = max_batch, max_tokens, max_pages, n_axes
        sizes = dict(q_indptr=max_batch + 1, kv_lens=max_batch, page_indptr=max_batch + 1, page_indices=max_pages,
                     positions=n_axes * max_tokens, token_req=max_tokens, cache_pos=max_tokens, row_slot=max_batch,
                     kv_indptr=max_batch + 1, logit_rows64=2 * max_batch)
        self.offsets, off = {}, 0
        for k, n in sizes.items():
            off = (off + 3) // 4 * 4   # 16-byte aligned sections
            self.offsets[k] = (off, n)
            off += n
        self.total = off
        self.cuda = torch.cuda.is_available() and self.device.type == "cuda"
        self.hosts = [torch.zeros(self.total, dtype=torch.int32, pin_memory=self.cuda) for _ in range(n_host)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.events = [None] * n_host
        self.cur = 0
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=self.device)

    def begin(self):
        """Next staging buffer (numpy view), free to be overwritten."""
        self.cur = (self.cur + 1) % len(self.hosts)
        ev = self.events[self.cur]
        if ev is not None:
            ev.synchronize()
        return self.hosts_np[self.cur]

    def d(self, name: str) -> torch.Tensor:
        o, n = self.offsets[name]
        return self.dev[o:o + n]

    def upload(self, used: int | None = None) -> None:
        self.dev.copy_(self.hosts[self.cur], non_blocking=True)
        io_counters.add_h2d(self.total * 4)
        if self.cuda:
            ev = self.events[self.cur] or torch.cuda.Event()
            ev.record()
            self.events[self.cur] = ev


class BatchedCacheManager:
    def __init__(self, config: KVCacheConfig, device, *, max_batch: int = 256, max_tokens: int = 16384,
                 n_pos_axes: int = 1, num_plan_slots: int = 2, alloc: PagedAllocationManager | None = None):
        self.config = config
        self.device = torch.device(device)
        self.alloc = alloc or PagedAllocationManager(config, device)
        max_pages_per_req = (config.max_seq_len + config.page_size - 1) // config.page_size
        self._max_pages = min(config.max_num_pages + max_batch, max_batch * max_pages_per_req)
        # plan slots = independent device plans (e.g. one for prefill, one for decode graphs)
        self._slots = [_PlanBuffers(device, max_batch, max_tokens, self._max_pages, n_pos_axes)
                       for _ in range(num_plan_slots)]
        self.n_pos_axes = n_pos_axes
        self._custom_advance: dict[str, int] = {}

    # ---- request lifecycle ----
    def add_request(self, request_id: str, labels: list[str] | None = None) -> None:
        self.alloc.add_request(request_id, labels)

    def remove_request(self, request_id: str) -> None:
        self.alloc.remove_request(request_id)
        self._custom_advance.pop(request_id, None)

    def seq_len(self, request_id: str, label: str = "main") -> int:
        return self.alloc.get_state(request_id, label).seq_len

    def set_custom_pos_advance(self, request_id: str, label: str, delta: int) -> None:
        """Rope position of the next token = seq_len + delta (multimodal spans that advance positions
        differently from their token count)."""
        self.alloc.get_state(request_id, label).pos_offset = delta

    def snapshot(self, request_id: str, src: str, dst: str) -> None:
        self.alloc.copy_label(request_id, src, dst)

    # ---- planning ----
    def plan(self, request_ids: list[str], q_lens: list[int], *, labels: list[str] | None = None,
             causal: bool = True, window: int = 0, write_cache: bool = True,
             custom_positions: torch.Tensor | None = None, row_slots: list[int] | None = None,
             pad_to_batch: int | None = None, lookahead_tokens: int = 0, group: int = 1,
             slot: int = 0, splits: int | None = None, pad_row_slot: int = 0,
             pad_to_tokens: int | None = None) -> BatchContext:
        """Reserve pages for the new tokens and write the device plan. Entries are (request, label) pairs.
        ``pad_to_batch`` pads with empty entries (one token, no keys, no cache write) up to a captured batch size;
        ``lookahead_tokens`` reserves pages for that many future decode tokens so that device-side advance can run
        ahead of the host. ``pad_row_slot`` is the sampler slot that padding rows use: it must belong to no request,
        because the captured step samples every row and updates the slot's seen-token mask and draw counter.
        ``pad_to_tokens`` (with ``pad_to_batch``, prefill buckets) also pads the TOKEN count: the last padding entry
        takes the missing tokens; the tile count and the longest query length are then those of the bucket, so that
        every plan of a bucket launches the same grids and kernel variants."""
        B = len(request_ids)
        labels = labels or ["main"] * B
        cfg = self.config
        ps = cfg.page_size
        if write_cache:
            self.alloc.alloc_batch([(r, lb, n + lookahead_tokens) for r, lb, n in zip(request_ids, labels, q_lens)])
        states = [self.alloc.get_state(r, lb) for r, lb in zip(request_ids, labels)]
        Bp = max(B, pad_to_batch or 0)
        pad_lens = [1] * (Bp - B)
        if pad_to_tokens is not None:
            missing = int(pad_to_tokens) - sum(q_lens) - len(pad_lens)
            if not pad_lens or missing < 0:
                raise ValueError("token padding needs a padding entry and a bucket at least as large as the batch")
            pad_lens[-1] += missing
        T = sum(q_lens) + sum(pad_lens)
        buf = self._slots[slot]
        if Bp > buf.max_batch or T > buf.max_tokens:
            raise ValueError(f"batch {Bp} / tokens {T} exceed the plan buffer ({buf.max_batch} / {buf.max_tokens})")
        hn = buf.begin()
        def sec(name):
            o, n = buf.offsets[name]
            return hn[o:o + n]
        qi, kl, pi, pidx = sec("q_indptr"), sec("kv_lens"), sec("page_indptr"), sec("page_indices")
        pos, treq, cpos = sec("positions").reshape(self.n_pos_axes, -1), sec("token_req"), sec("cache_pos")
        rslot, lrows, kvi = sec("row_slot"), sec("logit_rows64").view(np.int64), sec("kv_indptr")
        pad = Bp - B
        ql = np.asarray(list(q_lens) + pad_lens, dtype=np.int64)
        seq = np.asarray([st.seq_len for st in states], dtype=np.int64)
        poff = np.asarray([st.pos_offset for st in states], dtype=np.int64)
        qi[0] = 0
        np.cumsum(ql, out=qi[1:Bp + 1])
        kl[:B] = seq + (ql[:B] if write_cache else 0)
        kl[B:Bp] = 0
        npages = np.asarray([len(st.pages) for st in states] + [0] * pad, dtype=np.int64)
        pi[0] = 0
        np.cumsum(npages, out=pi[1:Bp + 1])
        npg = int(pi[Bp])
        if npg > buf.max_pages:
            raise ValueError("plan buffer page table overflow")
        if npg:
            pidx[:npg] = np.fromiter((pg for st in states for pg in st.pages), dtype=np.int32, count=npg)
        # per-token arrays: entry index, offset inside the entry
        ent = np.repeat(np.arange(Bp, dtype=np.int64), ql)
        within = np.arange(T, dtype=np.int64) - np.repeat(qi[:Bp].astype(np.int64), ql)
        real = ent < B
        seq_p = np.concatenate([seq, np.zeros(pad, dtype=np.int64)])
        poff_p = np.concatenate([poff, np.zeros(pad, dtype=np.int64)])
        tok_pos = np.where(real, seq_p[ent] + within, -1)
        pos[:, :T] = np.where(real, seq_p[ent] + poff_p[ent] + within, 0)[None, :]
        cpos[:T] = tok_pos
        treq[:T] = np.where(real, ent, -1) if write_cache else -1
        rslot[:B] = np.asarray(row_slots, dtype=np.int32) if row_slots is not None else np.arange(B, dtype=np.int32)
        rslot[B:Bp] = pad_row_slot
        lrows[:Bp] = qi[1:Bp + 1].astype(np.int64) - 1
        kvi[:Bp + 1] = 0
        max_kv = int(kl[:Bp].max()) if Bp else 0
        if custom_positions is not None:
            cp = custom_positions.reshape(-1, custom_positions.shape[-1]).to(torch.int32).cpu().numpy()
            pos[:cp.shape[0], :cp.shape[1]] = cp
            if cp.shape[0] < self.n_pos_axes:
                pos[cp.shape[0]:, :cp.shape[1]] = cp[0]
        buf.upload()
        if pad_to_tokens is not None:
            tpt = max(1, 128 // group)
            ntiles = (int(pad_to_tokens) + tpt - 1) // tpt + Bp      # upper bound over every plan of the bucket
        else:
            ntiles = attn_ops.count_q_tiles(list(q_lens) + pad_lens, group)
        if splits is None:
            splits = attn_ops.choose_splits(Bp, cfg.num_kv_heads, ntiles, max_kv) if max(q_lens, default=1) == 1 else 1
        plan = attn_ops.AttnPlan(q_indptr=buf.d("q_indptr"), kv_lens=buf.d("kv_lens"), batch=Bp, num_q_tokens=T,
                                 num_q_tiles=ntiles, page_indptr=buf.d("page_indptr"),
                                 page_indices=buf.d("page_indices"), splits=splits, causal=causal, window=window,
                                 max_q_len=int(pad_to_tokens) if pad_to_tokens is not None else max(list(q_lens) + [1]))
        ctx = BatchContext(plan=plan, positions=buf.d("positions").view(self.n_pos_axes, -1)[:, :T]
                           if self.n_pos_axes > 1 else buf.d("positions")[:T],
                           token_req=buf.d("token_req")[:T], cache_pos=buf.d("cache_pos")[:T],
                           logit_rows=buf.d("logit_rows64").view(torch.int64)[:Bp], row_slot=buf.d("row_slot")[:Bp],
                           kv_layers=self.alloc.kv_layers, num_tokens=T, batch=Bp, request_ids=list(request_ids),
                           labels=list(labels), q_lens=list(q_lens), write_cache=write_cache)
        return ctx

    def span_plan(self, ctx: BatchContext, spans: list[tuple[int, int, int]], group: int = 1):
        """A second, non-causal plan over row ranges of a batch that ``plan`` has just laid out (before the forward
        advances the sequence lengths): every span ``(entry, start, end)`` — rows ``start … end-1`` of that entry's new
        tokens — becomes an entry whose queries see the entry's cached keys and the new ones up to ``end``. A packed
        prompt runs its causal pass over all rows and then this pass over the spans that attend among themselves
        (the rows between an image's start and end markers). Returns (plan, int64 rows of the spans in the batch's
        token order); built from fresh device tensors, so it is not for captured graphs."""
        qi, kl, pi, pidx, rows, off = [0], [], [0], [], [], [0]
        for n in ctx.q_lens:
            off.append(off[-1] + n)
        for e, a, b in spans:
            if not (0 <= a < b <= ctx.q_lens[e]):
                raise ValueError(f"span {(e, a, b)} outside entry of {ctx.q_lens[e]} rows")
            st = self.alloc.get_state(ctx.request_ids[e], ctx.labels[e])
            qi.append(qi[-1] + (b - a))
            kl.append(st.seq_len + b)
            pidx += list(st.pages)
            pi.append(len(pidx))
            rows += range(off[e] + a, off[e] + b)
        i32 = dict(dtype=torch.int32, device=self.device)
        lens = [b - a for _, a, b in spans]
        plan = attn_ops.AttnPlan(q_indptr=torch.tensor(qi, **i32), kv_lens=torch.tensor(kl, **i32), batch=len(spans),
                                 num_q_tokens=qi[-1], num_q_tiles=attn_ops.count_q_tiles(lens, group),
                                 page_indptr=torch.tensor(pi, **i32), page_indices=torch.tensor(pidx, **i32), splits=1,
                                 causal=False, window=0, max_q_len=max(lens))
        return plan, torch.tensor(rows, dtype=torch.int64, device=self.device)

    def plan_snapshot(self, slot: int) -> torch.Tensor:
        return self._slots[slot].dev.clone()

    def plan_restore(self, slot: int, saved: torch.Tensor) -> None:
        self._slots[slot].dev.copy_(saved)

    def advance_seq_lens(self, ctx: BatchContext, counts: list[int] | None = None) -> None:
        """Host-side bookkeeping after a forward that wrote K/V: seq_len += tokens written."""
        if not ctx.write_cache:
            return
        counts = counts or ctx.q_lens
        for r, lb, n in zip(ctx.request_ids, ctx.labels, counts):
            self.alloc.get_state(r, lb).seq_len += n

    def advance_on_device(self, ctx: BatchContext, input_ids: torch.Tensor | None, sampled: torch.Tensor | None) -> None:
        """Decode only (one token per entry): kv_lens += 1, positions/cache slots move on, next input ids = the
        sampled tokens. Padded entries (kv_len 0 and token_req -1) are advanced too but stay without cache
        writes. Part of the captured step."""
        B = ctx.batch
        ew_ops.advance_decode(ctx.plan.kv_lens[:B], ctx.positions, ctx.cache_pos[:B], input_ids, sampled)
