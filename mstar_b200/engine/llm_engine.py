"""Single-node autoregressive engine: continuous batching over the paged KV pool with CUDA-graph decode.

Scheduling model. Every running request owns a *row* of the decode batch for its whole life (rows of finished
requests become padding until they are reused), so the decode step's static buffers never need compaction:
``input_ids[row]`` is written on the device by the previous step's sampler, the host only re-uploads the small
plan (lengths, page tables) each step. A step is captured once per batch-size bucket and replayed; the host runs
one step ahead of the GPU and reads sampled tokens from pinned memory with one step of lag, so stop conditions
are found late by one step (the extra token is dropped), like the reference's 1-deep speculation.

Prefill packs the waiting requests' prompts into one varlen forward (chunked to ``max_prefill_tokens``), samples
their first token and drops it into their row.

Reference counterparts: ``KVCacheEngine`` execute paths (mstar/engine/kv_cache_engine.py:517-781,897-1046),
``CudaGraphRunner`` BASIC_BATCHED decode capture/replay with double-buffered slots and in-graph sampling
(mstar/engine/cuda_graph_runner.py:585-850,1308-1534,1866-1989), micro-scheduler batch limits
(mstar/worker/micro_scheduler.py:212-340).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

import torch

from ..ops import _lib
from ..ops.sampling import SamplerState, SamplingConfig
from .cache_manager import BatchedCacheManager
from .kv_store import AllocationFailedError, KVCacheConfig

DEFAULT_CAPTURE_SIZES = [1, 2, 4, 8, 16, 32, 64, 128, 256]


@dataclass
class GenRequest:
    request_id: str
    prompt_ids: list[int]
    max_new_tokens: int
    sampling: SamplingConfig
    eos_ids: tuple[int, ...] = ()
    seed: int | None = None
    # runtime
    row: int = -1
    output_ids: list[int] = field(default_factory=list)
    dispatched: int = 0              # decode steps launched for this request (incl. the prefill sample)
    finished: bool = False
    t_arrive: float = 0.0
    t_first_token: float | None = None
    t_done: float | None = None


class _InFlight:
    """A launched step whose sampled tokens have not been read yet."""
    __slots__ = ("event", "host_tokens", "rows", "kind")

    def __init__(self, event, host_tokens, rows, kind):
        # rows: list of (row, request) — the request object, because a row may change hands before the read
        self.event, self.host_tokens, self.rows, self.kind = event, host_tokens, rows, kind


class LLMEngine:
    def __init__(self, model, kv_config: KVCacheConfig, device, *, max_batch: int = 64,
                 max_prefill_tokens: int = 8192, use_cuda_graphs: bool | None = None,
                 capture_sizes: list[int] | None = None, track_seen: bool = False, logits_dtype=torch.float32,
                 on_token=None):
        self.model = model
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.max_batch = max_batch
        self.max_prefill_tokens = max_prefill_tokens
        self.cfg = model.cfg
        self.group = max(1, model.layers[0].self_attn.Hq // model.layers[0].self_attn.Hkv)
        self.cache = BatchedCacheManager(kv_config, device, max_batch=max_batch,
                                         max_tokens=max(max_prefill_tokens, max_batch) + max_batch,
                                         n_pos_axes=self.cfg.n_pos_axes)
        self.sampler = SamplerState(max_batch, self.cfg.vocab_size, device, track_seen=track_seen)
        self.logits_dtype = logits_dtype
        self.use_graphs = self.cuda if use_cuda_graphs is None else (use_cuda_graphs and self.cuda)
        self.capture_sizes = sorted(s for s in (capture_sizes or DEFAULT_CAPTURE_SIZES) if s <= max_batch)
        if not self.capture_sizes or self.capture_sizes[-1] < max_batch:
            self.capture_sizes.append(max_batch)
        self.on_token = on_token
        # static decode buffers
        self.input_ids = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self.sampled = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.launches_per_decode_graph: dict[int, int] = {}   # this library's kernels recorded per captured step
        self._rows: list[GenRequest | None] = [None] * max_batch
        self.waiting: deque[GenRequest] = deque()
        self.requests: dict[str, GenRequest] = {}
        self._inflight: deque[_InFlight] = deque()
        self._host_bufs = [torch.zeros(max_batch, dtype=torch.int64, pin_memory=self.cuda) for _ in range(4)]
        self._host_i = 0
        self.stats = dict(decode_steps=0, prefill_calls=0, prefill_tokens=0, graph_replays=0, tokens_out=0,
                          h2d_bytes=0, d2h_bytes=0, kernel_launches=0)

    # ------------------------------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt_ids: list[int], max_new_tokens: int,
                    sampling: SamplingConfig | None = None, eos_ids: tuple[int, ...] = (), seed: int | None = None):
        req = GenRequest(request_id, list(prompt_ids), max_new_tokens,
                         sampling or SamplingConfig(self.cfg.vocab_size, temperature=0.0), tuple(eos_ids), seed)
        req.t_arrive = time.perf_counter()
        self.requests[request_id] = req
        self.waiting.append(req)
        return req

    def abort(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return
        if req in self.waiting:
            self.waiting.remove(req)
        self._finish(req)

    def has_work(self) -> bool:
        return bool(self.waiting) or any(r is not None for r in self._rows) or bool(self._inflight)

    @property
    def num_running(self) -> int:
        return sum(r is not None for r in self._rows)

    # ------------------------------------------------------------------------------------------------
    def _finish(self, req: GenRequest) -> None:
        if req.finished:
            return
        req.finished = True
        req.t_done = time.perf_counter()
        if req.row >= 0:
            self._rows[req.row] = None
        self.cache.remove_request(req.request_id)
        self.sampler.release(req.request_id)

    def _free_rows(self) -> list[int]:
        return [i for i, r in enumerate(self._rows) if r is None]

    def _pages_for(self, n_tokens: int) -> int:
        ps = self.cache.config.page_size
        return (n_tokens + ps - 1) // ps

    # ---- prefill ----
    def _admit(self) -> list[GenRequest]:
        """Take waiting requests while rows, prefill-token budget and pages last."""
        free = self._free_rows()
        admitted, tokens = [], 0
        pages_left = self.cache.alloc.num_free_pages
        while self.waiting and free:
            req = self.waiting[0]
            n = len(req.prompt_ids)
            need = self._pages_for(n + 1)
            if admitted and tokens + n > self.max_prefill_tokens:
                break
            if need > pages_left:
                break
            self.waiting.popleft()
            pages_left -= need
            tokens += n
            req.row = free.pop(0)
            self._rows[req.row] = req
            admitted.append(req)
        return admitted

    @torch.no_grad()
    def _prefill(self, reqs: list[GenRequest]) -> None:
        rids = [r.request_id for r in reqs]
        q_lens = [len(r.prompt_ids) for r in reqs]
        for r in reqs:
            self.cache.add_request(r.request_id)
            # the sampler slot is the decode row, so the decode graph samples with row == slot
            self.sampler.assign(r.request_id, r.sampling, seed=r.seed, slot=r.row)
        ctx = self.cache.plan(rids, q_lens, row_slots=[r.row for r in reqs], group=self.group, slot=1)
        ids = torch.tensor([t for r in reqs for t in r.prompt_ids], dtype=torch.int64)
        if self.cuda:
            ids = ids.pin_memory().to(self.device, non_blocking=True)
            self.stats["h2d_bytes"] += ids.numel() * 8 + self.cache._slots[1].total * 4
        logits = self.model(ctx, input_ids=ids)
        if logits.dtype != self.logits_dtype:
            logits = logits.to(self.logits_dtype)
        tok = self.sampler.sample(logits, ctx.row_slot)
        rows = torch.tensor([r.row for r in reqs], dtype=torch.int64, device=self.device)
        self.input_ids.index_copy_(0, rows, tok)
        self.cache.advance_seq_lens(ctx)
        for r in reqs:
            r.dispatched = 1
        self._push_inflight(tok, [(r.row, r) for r in reqs], "prefill")
        self.stats["prefill_calls"] += 1
        self.stats["prefill_tokens"] += sum(q_lens)

    # ---- decode ----
    def _decode_body(self, ctx) -> None:
        logits = self.model(ctx, input_ids=self.input_ids[:ctx.batch])
        self.sampler.sample(logits, ctx.row_slot, out=self.sampled[:ctx.batch], advance=False)
        self.sampler.offset[:ctx.batch] += 1
        self.input_ids[:ctx.batch].copy_(self.sampled[:ctx.batch])

    def _bucket(self, n_rows: int) -> int:
        for s in self.capture_sizes:
            if s >= n_rows:
                return s
        return self.capture_sizes[-1]

    @torch.no_grad()
    def _decode(self) -> None:
        active = [(i, r) for i, r in enumerate(self._rows) if r is not None and not r.finished
                  and r.dispatched < r.max_new_tokens]
        if not active:
            return
        n_rows = max(i for i, _ in active) + 1
        B = self._bucket(n_rows) if self.use_graphs else n_rows
        # rows without a live request are planned as padding: one token, no keys, no cache write
        rids, q_lens, slots = [], [], []
        live_rows = {i: r for i, r in active}
        # entries must be listed row by row; padding rows in between use a sentinel handled below
        try:
            ctx = self._plan_rows(live_rows, B)
        except AllocationFailedError:
            # out of pages: finish the youngest request's turn later; simplest policy is to stall admission and
            # drop the longest sequence to the waiting queue (its KV is released and will be recomputed)
            victim = max(live_rows.values(), key=lambda r: len(r.prompt_ids) + r.dispatched)
            self._preempt(victim)
            return
        if self.use_graphs:
            g = self._graphs.get(B)
            if g is None:
                g = self._capture(B, ctx)
            g.replay()
            self.stats["graph_replays"] += 1
        else:
            self._decode_body(ctx)
        for i, r in active:
            self.cache.alloc.get_state(r.request_id, "main").seq_len += 1
            r.dispatched += 1
        self._push_inflight(self.sampled[:B], list(active), "decode")
        self.stats["decode_steps"] += 1

    def _plan_rows(self, live_rows: dict[int, GenRequest], B: int):
        """Plan a decode step whose entry b is row b: live rows get their request, others are padding."""
        cm = self.cache
        alloc = cm.alloc
        alloc.alloc_batch([(r.request_id, "main", 1) for r in live_rows.values()])
        buf = cm._slots[0]
        hn = buf.begin()

        def sec(name):
            o, n = buf.offsets[name]
            return hn[o:o + n]
        import numpy as np
        qi, kl, pi, pidx = sec("q_indptr"), sec("kv_lens"), sec("page_indptr"), sec("page_indices")
        pos, treq, cpos = sec("positions").reshape(cm.n_pos_axes, -1), sec("token_req"), sec("cache_pos")
        rslot, lrows = sec("row_slot"), sec("logit_rows64").view(np.int64)
        qi[:B + 1] = np.arange(B + 1, dtype=np.int32)
        lrows[:B] = np.arange(B, dtype=np.int64)
        rslot[:B] = np.arange(B, dtype=np.int32)
        kl[:B] = 0
        treq[:B] = -1
        cpos[:B] = -1
        pos[:, :B] = 0
        npg = 0
        max_kv = 0
        counts = np.zeros(B, dtype=np.int64)
        for i, r in live_rows.items():
            st = alloc.get_state(r.request_id, "main")
            n = len(st.pages)
            counts[i] = n
            kl[i] = st.seq_len + 1
            treq[i] = i
            cpos[i] = st.seq_len
            pos[:, i] = st.seq_len + st.pos_offset
            max_kv = max(max_kv, st.seq_len + 1)
        pi[0] = 0
        np.cumsum(counts, out=pi[1:B + 1])
        for i, r in live_rows.items():
            st = alloc.get_state(r.request_id, "main")
            o = int(pi[i])
            pidx[o:o + len(st.pages)] = st.pages
        buf.upload()
        self.stats["h2d_bytes"] += buf.total * 4
        from ..ops import attention as attn_ops
        ntiles = B
        splits = self._graph_splits.get(B) if self.use_graphs and hasattr(self, "_graph_splits") else None
        if splits is None:
            splits = attn_ops.choose_splits(B, cm.config.num_kv_heads, ntiles, max_kv, sm_count=3 * 148)
        plan = attn_ops.AttnPlan(q_indptr=buf.d("q_indptr"), kv_lens=buf.d("kv_lens"), batch=B, num_q_tokens=B,
                                 num_q_tiles=ntiles, page_indptr=buf.d("page_indptr"),
                                 page_indices=buf.d("page_indices"), splits=splits, causal=True,
                                 window=self.cfg.sliding_window, max_q_len=1)
        from .cache_manager import BatchContext
        positions = buf.d("positions").view(cm.n_pos_axes, -1)[:, :B] if cm.n_pos_axes > 1 else buf.d("positions")[:B]
        return BatchContext(plan=plan, positions=positions, token_req=buf.d("token_req")[:B],
                            cache_pos=buf.d("cache_pos")[:B], logit_rows=buf.d("logit_rows64").view(torch.int64)[:B],
                            row_slot=buf.d("row_slot")[:B], kv_layers=alloc.kv_layers, num_tokens=B, batch=B)

    def _capture(self, B: int, ctx) -> torch.cuda.CUDAGraph:
        """Warm up (also sizes scratch buffers and configures kernels), then capture the decode step for batch B.
        The split-KV factor is frozen per bucket from the engine's max_seq_len so replays keep one grid."""
        from ..ops import attention as attn_ops
        if not hasattr(self, "_graph_splits"):
            self._graph_splits = {}
        splits = attn_ops.choose_splits(B, self.cache.config.num_kv_heads, B, self.cache.config.max_seq_len,
                                        sm_count=3 * 148)
        self._graph_splits[B] = splits
        ctx.plan.splits = splits
        attn_ops.reserve_scratch(self.device, B * self.model.layers[0].self_attn.Hq, self.cfg.head_dim, splits,
                                 B * self.cache.config.num_kv_heads)
        saved = (self.input_ids.clone(), self.sampler.offset.clone(),
                 None if self.sampler.seen is None else self.sampler.seen.clone())
        kv_backup = None
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_body(ctx)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            from ..ops import _counters
            c0 = _counters.get()
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                self._decode_body(ctx)
            self.launches_per_decode_graph[B] = _counters.get() - c0
        torch.cuda.current_stream().wait_stream(s)
        # warm-up runs wrote K/V at the planned slots (they are rewritten by the real step) and bumped sampler state
        self.input_ids.copy_(saved[0])
        self.sampler.offset.copy_(saved[1])
        if saved[2] is not None:
            self.sampler.seen.copy_(saved[2])
        del kv_backup
        self._graphs[B] = g
        return g

    def _preempt(self, req: GenRequest) -> None:
        """Release a request's KV and requeue it with its generated prefix as part of the prompt."""
        self._drain()
        if req.finished:          # the tokens still in flight completed it: nothing left to recompute
            return
        self._rows[req.row] = None
        self.cache.remove_request(req.request_id)
        self.sampler.release(req.request_id)
        req.prompt_ids = req.prompt_ids + req.output_ids
        req.max_new_tokens -= len(req.output_ids)
        req.output_ids_prefix = getattr(req, "output_ids_prefix", []) + req.output_ids
        req.output_ids = []
        req.row, req.dispatched = -1, 0
        self.waiting.appendleft(req)

    # ---- token readback ----
    def _push_inflight(self, tok: torch.Tensor, rows: list, kind: str) -> None:
        if self.cuda:
            host = self._host_bufs[self._host_i]
            self._host_i = (self._host_i + 1) % len(self._host_bufs)
            host[:tok.numel()].copy_(tok, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.stats["d2h_bytes"] += tok.numel() * 8
        else:
            host, ev = tok.clone(), None
        self._inflight.append(_InFlight(ev, host, rows, kind))

    def _collect(self, item: _InFlight) -> list[tuple[str, int]]:
        if item.event is not None:
            item.event.synchronize()
        out = []
        now = time.perf_counter()
        vals = item.host_tokens.tolist()
        for j, (row, req) in enumerate(item.rows):
            if req.finished or req.row != row:
                continue
            tok = vals[j] if item.kind == "prefill" else vals[row]
            req.output_ids.append(tok)
            if req.t_first_token is None:
                req.t_first_token = now
            self.stats["tokens_out"] += 1
            out.append((req.request_id, tok))
            if self.on_token is not None:
                self.on_token(req, tok)
            hit_eos = (not req.sampling.ignore_eos) and tok in req.eos_ids
            if hit_eos or len(req.output_ids) >= req.max_new_tokens:
                self._finish(req)
        return out

    def _drain(self) -> list[tuple[str, int]]:
        out = []
        while self._inflight:
            out += self._collect(self._inflight.popleft())
        return out

    # ------------------------------------------------------------------------------------------------
    def step(self, max_lag: int = 1) -> list[tuple[str, int]]:
        """Admit + prefill waiting requests, launch one decode step, read back tokens of steps older than
        ``max_lag``. Returns the (request_id, token) pairs read in this call."""
        out = []
        launched_before = self.stats["decode_steps"] + self.stats["prefill_calls"]
        admitted = self._admit()
        if admitted:
            self._prefill(admitted)
        self._decode()
        while len(self._inflight) > max_lag:
            out += self._collect(self._inflight.popleft())
        launched = self.stats["decode_steps"] + self.stats["prefill_calls"] - launched_before
        if launched == 0:
            # nothing new could start (rows are waiting for their last tokens to be read): read everything
            out += self._drain()
        return out

    def run_to_completion(self) -> dict[str, list[int]]:
        while self.has_work():
            self.step()
        return {rid: getattr(r, "output_ids_prefix", []) + r.output_ids for rid, r in self.requests.items()}

    def check_status(self) -> None:
        """Raise if a kernel's bounded wait ran out since the last check."""
        if self.cuda:
            code, block, a0, a1 = _lib.read_status(clear=True)
            if code:
                raise RuntimeError(f"kernel status {code:#x} (block {block}, aux {a0}, {a1})")
