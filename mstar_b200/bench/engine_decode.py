"""Device-timed decode steps on the SERVING engine: the same ``KVCacheEngine`` + LLM submodule that a worker builds
for the ``LLM`` node of the Orpheus deployment, driven the way the worker drives it (``NodeBatch`` ->
``launch_batch`` / ``collect_batch``; decode bursts; the continuation of a burst queued while the burst runs).
``bench.py`` uses it for its CUDA-event number; the served number goes through the whole server instead.

A step is one decode step of every running request. Every step's plan comes from pinned host memory (one upload
per burst) and every step's sampled ids go back to pinned host memory, as in serving.
"""
from __future__ import annotations

import torch

from ..engine.base import NodeBatch
from ..models.orpheus import OrpheusModel
from ..ops import _counters
from ..utils.ipc_format import CurrentForwardPassInfo
from ..worker.engine_manager import EngineManager


class EngineDecodeHarness:
    def __init__(self, device, concurrency: int = 64, max_ctx: int = 2048, tp_group=None, page_size: int = 128,
                 sampling: dict | None = None):
        self.device = torch.device(device)
        pages = concurrency * ((max_ctx + page_size - 1) // page_size) + 64
        self.model = OrpheusModel(skip_weight_loading=True, page_size=page_size, max_num_pages=pages)
        self.em = EngineManager(self.model, self.device, ["LLM"], tp_group=tp_group, max_batch=concurrency)
        self.eng = self.em.engine_for("LLM")
        self.sampling = sampling or dict(temperature=0.6, top_p=0.8, repetition_penalty=1.3, ignore_eos=True)
        self.infos: dict[str, CurrentForwardPassInfo] = {}
        self.tok: dict[str, torch.Tensor] = {}
        self.order: list[str] = []
        self.steps_done = 0

    def _info(self, rid: str, walk: str, remaining: int) -> CurrentForwardPassInfo:
        fi = self.infos.get(rid)
        if fi is None:
            fi = self.infos[rid] = CurrentForwardPassInfo(rid, walk, sampling_config={"main": dict(self.sampling)})
        fi.graph_walk = walk
        fi.step_metadata = {"_loop_remaining": remaining}
        return fi

    def prefill(self, prompts: dict[str, list[int]], max_tokens: int = 12288) -> None:
        """Real prefill of every prompt, in packed batches of at most ``max_tokens`` tokens."""
        batch, n = [], 0
        items = list(prompts.items())
        for i, (rid, ids) in enumerate(items):
            batch.append((rid, ids))
            n += len(ids)
            nxt = len(items[i + 1][1]) if i + 1 < len(items) else 0
            if i + 1 == len(items) or n + nxt > max_tokens:
                rids = [r for r, _ in batch]
                nb = NodeBatch("LLM", "prefill", rids,
                               {r: {"input_ids": [torch.tensor(x, dtype=torch.int64)]} for r, x in batch},
                               {r: self._info(r, "prefill", 1) for r in rids})
                out = self.eng.execute_batch(nb)
                if out.failed_requests or out.allocation_failed:
                    raise RuntimeError(f"prefill failed: {out.failed_requests or out.timings}")
                for r in rids:
                    self.tok[r] = out.outputs[r]["tok"]
                    self.order.append(r)
                batch, n = [], 0

    def decode(self, steps: int):
        """``steps`` decode steps of all requests as bursts, each burst queued before the previous one is read back.
        Returns (CUDA-event milliseconds over all bursts, bursts run, this library's kernel launches)."""
        eng = self.eng
        rids = list(self.order)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c_graph0, launches = eng.graph_hits, 0
        left, pend_prev, bursts, first = steps, None, 0, True
        ev0.record()
        while left > 0:
            infos = {r: self._info(r, "decode", left) for r in rids}
            if first:
                nb = NodeBatch("LLM", "decode", rids, {r: {"tok": [self.tok[r]]} for r in rids}, infos)
            else:
                nb = NodeBatch("LLM", "decode", rids, {r: {} for r in rids}, infos, speculative=True)
            c0 = _counters.get()
            pend = eng.launch_batch(nb)
            launches += _counters.get() - c0            # launches outside the captured step (plan, copies)
            if pend.planned is None or pend.out.allocation_failed:
                raise RuntimeError(f"decode launch failed: {pend.out.failed_requests or pend.out.timings}")
            if pend_prev is not None:
                self._collect(pend_prev, rids)
            pend_prev, first = pend, False
            left -= pend.iterations
            bursts += 1
        ev1.record()
        self._collect(pend_prev, rids)
        torch.cuda.synchronize(self.device)
        replays = eng.graph_hits - c_graph0
        per_graph = max(eng.launches_per_graph.values()) if eng.launches_per_graph else 0
        self.steps_done += steps
        return ev0.elapsed_time(ev1), bursts, launches + replays * per_graph

    def _collect(self, pend, rids) -> None:
        out = self.eng.collect_batch(pend)
        bad = self.eng.check_batch_status(out)
        if bad or out.failed_requests:
            raise RuntimeError(f"decode failed: {bad or out.failed_requests}")
        for r in rids:
            self.tok[r] = out.outputs[r]["tok"]
