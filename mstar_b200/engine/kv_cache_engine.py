"""Engine for autoregressive nodes over the paged KV pool: owns the pool, the batch planner, the sampler and the
CUDA-graph buckets of its nodes' decode steps.

Dispatch per batch: captured graph (all entries decode one token, bucket available) > batched eager (packed
varlen forward) > per-request fallback. Allocation failures never escape as exceptions: the batch comes back with
``allocation_failed`` so the worker can offload a victim to the host pool or hold the requests.

Reference counterparts: ``KVCacheEngine`` (mstar/engine/kv_cache_engine.py:136-1356: load_model :177-294, warmup
:357-455, _execute_batched :517-635, _can_use_cuda_graph :701-781, execute_batch envelope :818-869, prepare_batch
:897-999, execute_forward with the TP barrier :1001-1046, offload :1294-1349), BASIC_BATCHED decode graphs and
in-graph sampling (mstar/engine/cuda_graph_runner.py:769-850,1308-1534,1866-1989).
"""
from __future__ import annotations

import os

import torch

from ..models.submodule_base import BATCHED_LOGITS, ModelInputsFromEngine
from ..ops import _lib
from ..ops import attention as attn_ops
from ..ops.sampling import SamplerState, SamplingConfig
from ..utils import io_counters
from .base import BaseEngine, NodeBatch, NodeOutput, PendingBatch, PreparedBatch
from .cache_manager import BatchedCacheManager
from .kv_store import AllocationFailedError, KVCacheConfig

CAPTURE_BATCH_SIZES = [1, 2, 4, 8, 16, 32, 64]
# prefill graphs: (batch bucket, token bucket) pairs; a packed prompt batch is padded with empty entries, the last
# of which takes the missing tokens
PREFILL_TOKEN_BUCKETS = [128, 256, 512, 1024, 2048]


class KVCacheEngine(BaseEngine):
    def __init__(self, node_names, device, kv_config: KVCacheConfig, *, vocab_size: int, max_batch: int = 64,
                 max_tokens: int = 16384, n_pos_axes: int = 1, group: int = 1, use_cuda_graphs: bool | None = None,
                 tp_group=None, track_seen: bool = True, decode_burst: int = 1):
        super().__init__(node_names, device)
        # decode burst: one node execution replays the captured decode step up to this many times back to back
        # (sampled tokens feed the next replay on the device), so the host-side cost of scheduling, routing and
        # bookkeeping is paid once per burst instead of once per token
        self.decode_burst = max(1, int(os.environ.get("MSTAR_DECODE_BURST", decode_burst)))
        self._burst_buf = torch.zeros((self.decode_burst, max_batch), dtype=torch.int64, device=torch.device(device))
        # sampled ids travel to the host through a ring of pinned buffers with an asynchronous copy behind the last
        # replay, so a following (speculative) batch can be queued before this one's tokens are read
        _cuda = torch.device(device).type == "cuda"
        self._host_ring = [torch.zeros((self.decode_burst, max_batch), dtype=torch.int64, pin_memory=_cuda)
                           for _ in range(4)]
        self._host_i = 0
        self._last_graph_key = None       # (node, walk, bucket, request ids) of the last captured-step execution
        # device time of the captured decode steps (CUDA events around each burst), kept only when statistics are on
        self._time_steps = _cuda and bool(os.environ.get("MSTAR_WORKER_STATS") or os.environ.get("MSTAR_WORKER_STATS_DIR"))
        self.decode_device_ms, self.decode_steps = 0.0, 0
        self.kv_config = kv_config
        self.cache = BatchedCacheManager(kv_config, device, max_batch=max_batch, max_tokens=max_tokens + max_batch,
                                         n_pos_axes=n_pos_axes)
        self.sampler = SamplerState(max_batch * 2 + 1, vocab_size, device, track_seen=track_seen, reserve_pad_slot=True)
        self.max_batch, self.group = max_batch, group
        self.tp_group = tp_group
        self.use_graphs = (self.device.type == "cuda") if use_cuda_graphs is None else (use_cuda_graphs and self.device.type == "cuda")
        # CPU stand-in for captured graphs (tests of the bucketed decode path and of decode bursts without a GPU):
        # "capture" keeps the step closure, "replay" calls it
        self.emulate_graphs = self.device.type != "cuda" and bool(os.environ.get("MSTAR_EMULATE_GRAPHS"))
        if self.emulate_graphs and use_cuda_graphs is not False:
            self.use_graphs = True
        self._graphs: dict[tuple, tuple] = {}
        self.launches_per_graph: dict[tuple, int] = {}     # this library's kernels recorded in each captured step
        self._static_ids = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self._static_prefill_ids = torch.zeros(PREFILL_TOKEN_BUCKETS[-1], dtype=torch.int64, device=self.device)
        # Opt-in (MSTAR_PREFILL_GRAPHS=1; the CPU stand-in for graphs always takes the path, so the tests cover it):
        # a bucket's graph is captured at its first use, and under a burst of arrivals that capture lands inside the
        # requests' time to first token (served TTS, 64 streams: first audio 304 ms p50 with it, 200 - 257 ms without)
        # while the replayed prefill saves only launch time, which a 64-request prefill does not wait for.
        self.prefill_graphs = os.environ.get("MSTAR_PREFILL_GRAPHS", "1" if self.emulate_graphs else "0") != "0"
        self.prefill_graph_hits = 0
        self._static_tok = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self.graph_hits = 0
        self.graph_misses: dict[str, int] = {}
        self.states: dict[str, dict] = {}

    # ---- request lifecycle ----
    def add_request(self, request_id: str, fwd_info) -> None:
        if not self.cache.alloc.has_request(request_id):
            self.cache.add_request(request_id)
        sc = (fwd_info.sampling_config or {}).get("main", {})
        cfg = SamplingConfig(self.sampler.vocab_size, **{k: sc[k] for k in
                             ("temperature", "top_k", "top_p", "repetition_penalty", "ignore_eos") if k in sc})
        self.sampler.assign(request_id, cfg, seed=fwd_info.random_seed or None)

    def remove_request(self, request_id: str) -> None:
        self.cache.remove_request(request_id)
        self.sampler.release(request_id)
        self.states.pop(request_id, None)
        super().remove_request(request_id)

    def get_per_label_seq_info(self, request_id: str) -> dict:
        return self.cache.alloc.get_per_label_seq_info(request_id)

    # ---- prefill / decode disaggregation ----
    def import_kv_from(self, src: "KVCacheEngine", request_id: str, fwd_info) -> int:
        """Pull a request's K/V pages (device-to-device, over NVLink between GPUs) and sampler state from the
        engine that ran its prefill. Returns the number of pages moved."""
        from .kv_store import PeerKVTransfer
        desc = src.cache.alloc.export_descriptor(request_id)
        self.add_request(request_id, fwd_info)
        PeerKVTransfer(self.cache.alloc).pull(request_id, src.cache.alloc.kv_layers, desc)
        if request_id in src.sampler._slot_of:
            a, b = src.sampler.slot(request_id), self.sampler.slot(request_id)
            self.sampler.offset[b] = src.sampler.offset[a].to(self.device)
            if self.sampler.seen is not None and src.sampler.seen is not None:
                self.sampler.seen[b] = src.sampler.seen[a].to(self.device)
        return sum(len(d["pages"]) for d in desc.values())

    def export_kv(self, request_id: str) -> tuple[dict, dict[str, torch.Tensor]]:
        """The hand-off of a request to a pool in ANOTHER process: per label the pages gathered into one tensor
        ``[layers, pages, 2, kv_heads, page, head_dim]`` (sent like any tensor edge: a CUDA IPC handle between GPU
        processes, the shared-memory arena between CPU ones), plus page counts, lengths and the sampler's state."""
        desc = self.cache.alloc.export_descriptor(request_id)
        meta: dict = {"labels": {}, "sampler": None}
        tensors: dict[str, torch.Tensor] = {}
        for label, d in desc.items():
            meta["labels"][label] = dict(n_pages=len(d["pages"]), seq_len=d["seq_len"], pos_offset=d["pos_offset"])
            if d["pages"]:
                idx = torch.tensor(d["pages"], dtype=torch.long, device=self.device)
                tensors[f"kv:{label}"] = torch.stack([layer.index_select(0, idx) for layer in self.cache.alloc.kv_layers])
        if request_id in self.sampler._slot_of:
            a = self.sampler.slot(request_id)
            meta["sampler"] = dict(offset=int(self.sampler.offset[a].item()))
            if self.sampler.seen is not None:
                tensors["sampler:seen"] = self.sampler.seen[a].clone()
        return meta, tensors

    def import_kv(self, request_id: str, fwd_info, meta: dict, tensors: dict[str, torch.Tensor]) -> int:
        """Counterpart of ``export_kv`` on the receiving pool. Returns the number of pages stored."""
        self.add_request(request_id, fwd_info)
        alloc = self.cache.alloc
        moved = 0
        for label, d in meta["labels"].items():
            alloc.reset_label(request_id, label)
            st = alloc.get_state(request_id, label)
            if d["n_pages"]:
                st.pages = alloc.allocator.allocate(d["n_pages"])
                di = torch.tensor(st.pages, dtype=torch.long, device=self.device)
                t = tensors[f"kv:{label}"].to(self.device)
                for li, layer in enumerate(alloc.kv_layers):
                    layer[di] = t[li].to(layer.dtype)
                moved += d["n_pages"]
            st.seq_len, st.pos_offset = d["seq_len"], d["pos_offset"]
        if meta.get("sampler") is not None:
            b = self.sampler.slot(request_id)
            self.sampler.offset[b] = meta["sampler"]["offset"]
            if self.sampler.seen is not None and "sampler:seen" in tensors:
                self.sampler.seen[b] = tensors["sampler:seen"].to(self.device)
        return moved

    # ---- offload surface ----
    def can_offload(self) -> bool:
        return self.cache.alloc.cpu_pool is not None

    def offload_request(self, request_id: str) -> int:
        return self.cache.alloc.offload_request(request_id)

    def pages_of(self, request_id: str) -> int:
        return self.cache.alloc.pages_of(request_id)

    # ---- template steps ----
    def launch_batch(self, batch: NodeBatch) -> PendingBatch:
        try:
            return super().launch_batch(batch)
        except AllocationFailedError as e:
            out = NodeOutput(batch.node_name, batch.graph_walk, allocation_failed=True,
                             allocation_failed_requests=list(batch.request_ids))
            out.timings["allocation_error"] = str(e)
            return PendingBatch(batch, out)

    def can_speculate(self, node_name: str, graph_walk: str) -> bool:
        """The captured decode step leaves the sampled ids as its own next input and the plan advanced on the
        device, so iteration N+1 of a decode loop needs nothing from the host but page reservations."""
        sub = self.submodules.get(node_name)
        return bool(self.use_graphs and sub is not None and sub.can_use_cuda_graphs(graph_walk)
                    and self._last_graph_key is not None and self._last_graph_key[:2] == (node_name, graph_walk))

    def prepare_batch(self, batch: NodeBatch) -> PreparedBatch:
        for rid in batch.request_ids:
            if rid not in self.sampler._slot_of:
                self.add_request(rid, batch.fwd_infos[rid])
            if self.cache.alloc.is_offloaded(rid):
                self.cache.alloc.reload_request(rid)      # may raise AllocationFailedError -> envelope
        return super().prepare_batch(batch)

    def plan(self, prepared: PreparedBatch):
        b = prepared.batch
        sub = self.submodules[b.node_name]
        if hasattr(sub, "custom_plan"):
            # nodes that plan their own entries (several cache labels per request, reads without writes, ...);
            # None = this walk uses the default planning below
            ctx = sub.custom_plan(self.cache, b.graph_walk, prepared)
            if ctx is not None:
                prepared.ctx, prepared.bucket, prepared.q_lens = ctx, None, list(ctx.q_lens)
                return prepared
        q_lens = [1 if b.speculative else max(1, ni.input_seq_len) for ni in prepared.node_inputs]
        labels = [sub.get_needed_cache_labels(b.graph_walk, b.fwd_infos[r])[0] for r in prepared.request_ids]
        slots = [self.sampler.slot(r) for r in prepared.request_ids]
        decode = all(q == 1 for q in q_lens)
        B = len(q_lens)
        bucket = None
        if decode and self.use_graphs and sub.can_use_cuda_graphs(b.graph_walk):
            bucket = next((s for s in CAPTURE_BATCH_SIZES if s >= B and s <= self.max_batch), None)
            if bucket is None:
                self.graph_misses["batch larger than the largest bucket"] = self.graph_misses.get("batch larger than the largest bucket", 0) + 1
        token_bucket = None
        if (not decode and self.use_graphs and self.prefill_graphs and not b.speculative
                and sub.can_use_cuda_graphs(b.graph_walk) and sub.can_graph_prefill(b.graph_walk)
                and all(ni.custom_pos_ids is None and ni.input_ids is not None and ni.input_embeds is None
                        for ni in prepared.node_inputs)):
            # prefill replayed from a graph: smallest (batch, token) bucket with room for one padding entry
            T = sum(q_lens)
            bp = next((s_ for s_ in CAPTURE_BATCH_SIZES if s_ > B and s_ <= self.max_batch), None)
            tb = next((t_ for t_ in PREFILL_TOKEN_BUCKETS if bp is not None and t_ >= T + (bp - B)), None)
            if bp is not None and tb is not None:
                bucket, token_bucket = bp, tb
        if bucket is None and self.use_graphs:
            why = "prefill / multi-token step" if not decode else "node opted out"
            self.graph_misses[why] = self.graph_misses.get(why, 0) + 1
        custom = None
        if any(ni.custom_pos_ids is not None for ni in prepared.node_inputs):
            custom = torch.cat([ni.custom_pos_ids.reshape(ni.custom_pos_ids.shape[0] if ni.custom_pos_ids.dim() > 1 else 1, -1)
                                for ni in prepared.node_inputs], dim=-1)
        splits = None
        burst = 1
        if token_bucket is not None:
            splits = 1
        elif bucket is not None:
            splits = attn_ops.choose_splits(bucket, self.kv_config.num_kv_heads, bucket, self.kv_config.max_seq_len,
                                            sm_count=3 * 148)
            if self.decode_burst > 1 and token_bucket is None:       # no request may run past its loop budget inside the burst
                burst = max(1, min([self.decode_burst] + [int(ni.kwargs.get("_loop_remaining", 1))
                                                           for ni in prepared.node_inputs]))
        # decode buckets live in plan slot 0 (the captured decode step advances it on the device), everything else,
        # prefill buckets included, in slot 1
        ctx = self.cache.plan(prepared.request_ids, q_lens, labels=labels, row_slots=slots, pad_to_batch=bucket,
                              group=self.group, slot=0 if (bucket is not None and token_bucket is None) else 1,
                              custom_positions=custom, splits=splits, lookahead_tokens=burst - 1,
                              pad_row_slot=self.sampler.pad_slot, pad_to_tokens=token_bucket)
        prepared.ctx, prepared.bucket, prepared.q_lens, prepared.burst = ctx, bucket, q_lens, burst
        prepared.token_bucket = token_bucket
        return prepared

    def _forward_logits(self, sub, walk, ei, node_inputs):
        outs = sub.forward_batched(walk, ei, node_inputs)
        return outs

    def execute_forward(self, planned: PreparedBatch):
        b = planned.batch
        sub = self.submodules[b.node_name]
        ctx = planned.ctx
        if self.tp_group is not None and getattr(self.tp_group, "symm", None) is not None:
            self.tp_group.symm.barrier()
        ei = ModelInputsFromEngine(planned.request_ids, b.fwd_infos, cache_manager=self.cache, batch_context=ctx,
                                   sampler=self.sampler,
                                   per_request_states={r: self.states.setdefault(r, {}) for r in planned.request_ids})
        B = len(planned.request_ids)
        with torch.no_grad():
            if getattr(planned, "token_bucket", None) is not None:
                raw = self._replay_prefill(sub, b, ei, planned)
                self.cache.advance_seq_lens(ctx)
                return raw
            if planned.bucket is not None:
                sub.preprocess(b.graph_walk, ei, planned.node_inputs)
                key = (b.node_name, b.graph_walk, planned.bucket)
                run_key = key + (tuple(planned.request_ids),)
                if b.speculative:
                    # the previous execution (same rows, still running or just finished) left its sampled ids in the
                    # static input buffer: nothing to copy
                    if self._last_graph_key != run_key:
                        raise RuntimeError("speculative batch does not continue the engine's last execution")
                else:
                    ids = torch.cat([ni.input_ids.reshape(-1)[-1:] for ni in planned.node_inputs]).to(self.device)
                    self._static_ids[:B].copy_(ids)
                entry = self._graphs.get(key)
                if entry is None:
                    entry = self._capture(key, sub, b.graph_walk, ei, planned)
                self._last_graph_key = run_key
                k = getattr(planned, "burst", 1)
                evs = None
                if self._time_steps:
                    evs = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    evs[0].record()
                for j in range(k):
                    entry[0].replay()           # the graph leaves the plan advanced and the sampled ids as next input
                    self.graph_hits += 1
                    if k > 1:
                        self._burst_buf[j, :B].copy_(self._static_tok[:B])
                tokens = self._static_tok[:B].clone()
                raw = {"tokens": tokens, "extra": {k_: v[:B].clone() if isinstance(v, torch.Tensor) else v
                                                   for k_, v in entry[1].items()}}
                if evs is not None:
                    evs[1].record()
                    raw["timing"] = (evs, k)
                self._host_i = (self._host_i + 1) % len(self._host_ring)
                hb = self._host_ring[self._host_i]
                if k > 1:
                    raw["burst"] = self._burst_buf[:k, :B].t().contiguous()      # [B, k]
                    hb[:k, :B].copy_(self._burst_buf[:k, :B], non_blocking=True)
                    raw["burst_host"] = hb[:k, :B]
                    io_counters.add_d2h(k * B * 8)
                    self.cache.advance_seq_lens(ctx, counts=[k] * len(ctx.q_lens))
                    return raw
                hb[0, :B].copy_(tokens, non_blocking=True)
                raw["tokens_host"] = hb[0, :B]
                io_counters.add_d2h(B * 8)
            else:
                self._last_graph_key = None
                sub.preprocess(b.graph_walk, ei, planned.node_inputs)
                outs = sub.forward_batched(b.graph_walk, ei, planned.node_inputs)
                if isinstance(outs, list):           # one dict per request; logits rows (if any) are sampled
                    raw = {"per_request": outs}
                    rows = [(i, o.pop(BATCHED_LOGITS)) for i, o in enumerate(outs) if BATCHED_LOGITS in o]
                    if rows:
                        slots = torch.tensor([self.sampler.slot(planned.request_ids[i]) for i, _ in rows],
                                             dtype=torch.int32, device=self.device)
                        lg = torch.cat([r.reshape(1, -1) for _, r in rows]).float().contiguous()
                        toks = self.sampler.sample(lg, slots)
                        for (i, _), t in zip(rows, toks.tolist()):
                            outs[i]["new_token"] = torch.tensor([t], dtype=torch.int64)
                            outs[i]["new_token_host"] = t
                    outs = {}
                else:
                    raw = {"extra": {k: v for k, v in outs.items() if k != BATCHED_LOGITS}}
                if BATCHED_LOGITS in outs:
                    lg = outs[BATCHED_LOGITS]
                    if lg.dtype not in (torch.float32, torch.bfloat16):
                        lg = lg.float()
                    raw["tokens"] = self.sampler.sample(lg.contiguous(), ctx.row_slot[:lg.shape[0]])
        self.cache.advance_seq_lens(ctx)
        return raw

    def _replay_prefill(self, sub, b, ei, planned):
        """A packed prompt batch through the graph of its (batch, token) bucket: the prompt ids go into the static id
        buffer (padding tokens are id 0 on rows that write no K/V), the plan sits in its slot, the graph runs the
        model and samples every entry's last row."""
        ctx, Bp, Tb = planned.ctx, planned.bucket, planned.token_bucket
        B = len(planned.request_ids)
        self._last_graph_key = None
        sub.preprocess(b.graph_walk, ei, planned.node_inputs)
        ids = torch.cat([ni.input_ids.reshape(-1) for ni in planned.node_inputs])
        stage = torch.zeros(Tb, dtype=torch.int64)
        stage[:ids.numel()] = ids
        self._static_prefill_ids[:Tb].copy_(stage.to(self.device, non_blocking=True))
        key = (b.node_name, b.graph_walk, Bp, Tb)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(key, sub, b.graph_walk, ei, planned, ids_buf=self._static_prefill_ids[:Tb],
                                  plan_slot=1, advance=False)
        entry[0].replay()
        self.graph_hits += 1
        self.prefill_graph_hits += 1
        tokens = self._static_tok[:B].clone()
        raw = {"tokens": tokens, "extra": {k_: v[:B].clone() if isinstance(v, torch.Tensor) else v
                                           for k_, v in entry[1].items()}}
        self._host_i = (self._host_i + 1) % len(self._host_ring)
        hb = self._host_ring[self._host_i]
        hb[0, :B].copy_(tokens, non_blocking=True)
        raw["tokens_host"] = hb[0, :B]
        io_counters.add_d2h(B * 8)
        return raw

    def _capture(self, key, sub, walk, ei, planned, ids_buf=None, plan_slot=0, advance=True):
        """Capture model forward + sampling for one (node, walk, bucket). Inputs: the static id buffer and the
        plan slot; outputs: the static token buffer (+ any extra tensors the node returns)."""
        Bp = planned.bucket
        ctx = planned.ctx
        if self.device.type == "cuda":
            attn_ops.reserve_scratch(self.device, Bp * max(1, self.kv_config.num_qo_heads), self.kv_config.head_dim,
                                     max(1, ctx.plan.splits), Bp * self.kv_config.num_kv_heads)
        saved_off = self.sampler.offset.clone()
        saved_seen = None if self.sampler.seen is None else self.sampler.seen.clone()
        saved_plan = self.cache.plan_snapshot(plan_slot)
        saved_ids = self._static_ids.clone()
        ids_in = self._static_ids[:Bp] if ids_buf is None else ids_buf
        # device state that the node carries from step to step: the warm-up and capture runs must not advance it
        node_state = list(sub.capture_state()) if hasattr(sub, "capture_state") else []
        saved_state = [t.clone() for t in node_state]

        class _NI:      # node inputs view over the static id buffer
            pass

        def body():
            outs = sub.forward_graph(walk, ei, ids_in, ctx)
            self.sampler.sample(outs[BATCHED_LOGITS], ctx.row_slot, out=self._static_tok[:Bp], advance=False)
            self.sampler.offset.index_add_(0, ctx.row_slot.long(), torch.ones(Bp, dtype=torch.int64, device=self.device))
            if advance:
                # leave the device plan one token further and the sampled ids as the next input: a following replay
                # (decode burst) continues without the host; a following plan() simply rewrites the plan
                self.cache.advance_on_device(ctx, self._static_ids[:Bp], self._static_tok[:Bp])
            return {k: v for k, v in outs.items() if k != BATCHED_LOGITS}

        if self.emulate_graphs:
            class _Eager:
                def __init__(self, fn):
                    self.fn, self.extra = fn, {}

                def replay(self):
                    self.extra.update(self.fn())
            g = _Eager(body)
            extra = g.extra
            self._graphs[key] = (g, extra)
            return self._graphs[key]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                body()
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            from ..ops import _counters
            c0 = _counters.get()
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                extra = body()
            self.launches_per_graph[key] = _counters.get() - c0
        torch.cuda.current_stream().wait_stream(s)
        self.sampler.offset.copy_(saved_off)
        if saved_seen is not None:
            self.sampler.seen.copy_(saved_seen)
        self.cache.plan_restore(plan_slot, saved_plan)
        self._static_ids.copy_(saved_ids)
        for t, sv in zip(node_state, saved_state):
            t.copy_(sv)
        self._graphs[key] = (g, extra)
        return self._graphs[key]

    def postprocess(self, planned: PreparedBatch, raw, out: NodeOutput) -> None:
        b = planned.batch
        sub = self.submodules[b.node_name]
        tokens = raw.get("tokens")
        burst = raw.get("burst")
        if "timing" in raw:
            (e0, e1), k_ = raw["timing"]
            self.decode_device_ms += e0.elapsed_time(e1)
            self.decode_steps += k_
        # the ids were copied to pinned host memory behind the last replay (captured path): plain reads here
        burst_t = raw["burst_host"].t().contiguous() if burst is not None else None      # [B, k] host copy
        burst_host = burst_t.tolist() if burst_t is not None else None
        host_tokens = None
        if tokens is not None and burst is None:
            host_tokens = raw["tokens_host"].tolist() if "tokens_host" in raw else tokens.tolist()
        extra = raw.get("extra", {})
        nreq = len(planned.request_ids)
        per_row = {k: v for k, v in extra.items() if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == nreq}
        for i, (rid, ni) in enumerate(zip(planned.request_ids, planned.node_inputs)):
            try:
                fi = b.fwd_infos[rid]
                if "per_request" in raw:
                    r = dict(raw["per_request"][i])
                elif per_row:
                    r = {k: (per_row[k][i] if k in per_row else v) for k, v in extra.items()}
                else:
                    r = dict(extra)
                stops = None
                if burst_host is not None:
                    toks = burst_host[i]
                    n_valid = len(toks)
                    j = sub.first_stop_index(rid, fi, toks)      # cut the burst at the request's stop token
                    if j is not None:
                        n_valid = j + 1
                        stops = sub.check_stop(rid, fi, {"new_token_host": toks[j]})
                    if n_valid < len(toks):             # the positions written past the stop do not count
                        label = planned.ctx.labels[i] if i < len(planned.ctx.labels) else "main"
                        self.cache.alloc.get_state(rid, label).seq_len -= len(toks) - n_valid
                    r["new_token"] = burst[i, n_valid - 1:n_valid]
                    r["new_token_host"] = toks[n_valid - 1]
                    r["burst_host"] = toks[:n_valid]
                    r["burst_host_tensor"] = burst_t[i, :n_valid]
                    out.iterations[rid] = n_valid
                elif tokens is not None:
                    r["new_token"] = tokens[i:i + 1]
                    r["new_token_host"] = host_tokens[i]
                out.outputs[rid] = sub.postprocess(rid, fi, r, ni)
                if stops is None and burst_host is None:
                    stops = sub.check_stop(rid, fi, r)
                if stops:
                    out.stop_loops[rid] = set(stops)
            except Exception as e:  # noqa: BLE001
                out.failed_requests[rid] = f"postprocess failed: {e!r}"

    def check_status(self) -> None:
        if self.device.type == "cuda":
            code, block, a0, a1 = _lib.read_status(clear=True)
            if code:
                raise RuntimeError(f"kernel status {code:#x} (block {block}, aux {a0}, {a1})")
