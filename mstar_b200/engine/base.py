"""Engine contract: ``execute_batch = prepare -> plan -> execute_forward -> postprocess -> finalize``, with
per-request failure attribution and an allocation-failure envelope.

Reference counterparts: ``NodeBatch`` / ``PreparedBatch`` / ``PlannedBatch`` / ``NodeOutput`` and ``BaseEngine``
(mstar/engine/base.py:16-447; template :237-264, chunked execution :364-407).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..utils import io_counters


@dataclass
class NodeBatch:
    node_name: str
    graph_walk: str
    request_ids: list[str]
    inputs: dict[str, dict[str, list[torch.Tensor]]]     # request_id -> input name -> tensors
    fwd_infos: dict                                       # request_id -> CurrentForwardPassInfo
    # launched before the previous execution of the same node for the same requests was read back: its inputs are
    # the outputs that execution left on the device (a worker only sets this on engines that ``can_speculate``)
    speculative: bool = False


@dataclass
class PreparedBatch:
    batch: NodeBatch
    node_inputs: list = field(default_factory=list)      # per kept request, in order
    request_ids: list[str] = field(default_factory=list)
    failed_requests: dict[str, str] = field(default_factory=dict)


@dataclass
class NodeOutput:
    node_name: str
    graph_walk: str
    outputs: dict[str, dict[str, torch.Tensor]] = field(default_factory=dict)   # request_id -> edge name -> tensor
    stop_loops: dict[str, set] = field(default_factory=dict)                    # request_id -> loop names
    iterations: dict[str, int] = field(default_factory=dict)    # request_id -> loop iterations this execution covered
    failed_requests: dict[str, str] = field(default_factory=dict)
    allocation_failed: bool = False
    allocation_failed_requests: list[str] = field(default_factory=list)
    completion_event: object = None
    status_host: object = None        # pinned int32[4]: the device status word as of the end of this batch
    timings: dict = field(default_factory=dict)


@dataclass
class PendingBatch:
    """A batch whose GPU work is queued but whose results have not been read back: the hand-over between
    ``launch_batch`` (never waits for the GPU) and ``collect_batch`` (reads results; cheap once ``ready()``)."""
    batch: NodeBatch
    out: NodeOutput
    planned: object = None
    raw: object = None
    event: object = None              # recorded behind the batch's last kernel and result copy
    iterations: int = 1               # loop iterations every request of the batch covers (decode burst length)
    t_launch: tuple = ()

    def ready(self) -> bool:
        return self.event is None or self.event.query()


class BaseEngine:
    def __init__(self, node_names: list[str], device):
        self.node_names = list(node_names)
        self.device = torch.device(device)
        self.submodules: dict[str, object] = {}
        self.phase_s = dict(prepare=0.0, plan=0.0, forward=0.0, postprocess=0.0)

    # template ------------------------------------------------------------------------------------
    def execute_batch(self, batch: NodeBatch) -> NodeOutput:
        return self.collect_batch(self.launch_batch(batch))

    def launch_batch(self, batch: NodeBatch) -> PendingBatch:
        """prepare -> plan -> forward: queues the batch's GPU work and the copies of what the host will read, records
        an event behind them and returns without waiting. A worker launches the next batch (a speculative one
        included) while this one still runs, and calls ``collect_batch`` once ``pending.ready()``."""
        import time
        t0 = time.perf_counter()
        prepared = self.prepare_batch(batch)
        out = NodeOutput(batch.node_name, batch.graph_walk, failed_requests=dict(prepared.failed_requests))
        pend = PendingBatch(batch, out)
        if not prepared.request_ids:
            return pend
        t1 = time.perf_counter()
        planned = self.plan(prepared)
        t2 = time.perf_counter()
        pend.planned = planned
        pend.raw = self.execute_forward(planned)
        pend.iterations = max(1, int(getattr(planned, "burst", 1) or 1))
        self.finalize_batch(planned, out)
        pend.event = out.completion_event
        t3 = time.perf_counter()
        # host seconds of every phase (the forward's number is launch time only unless the phase synchronises)
        ph = self.phase_s
        ph["prepare"] += t1 - t0
        ph["plan"] += t2 - t1
        ph["forward"] += t3 - t2
        out.timings.update(prepare_s=t1 - t0, plan_s=t2 - t1, forward_s=t3 - t2)
        return pend

    def collect_batch(self, pend: PendingBatch) -> NodeOutput:
        """Wait for the batch (no wait when ``pend.ready()``), read its results and run the per-request
        postprocessing and stop checks."""
        import time
        out = pend.out
        if pend.planned is None:
            return out
        if pend.event is not None:
            pend.event.synchronize()
        t3 = time.perf_counter()
        self.postprocess(pend.planned, pend.raw, out)
        dt = time.perf_counter() - t3
        self.phase_s["postprocess"] += dt
        out.timings["postprocess_s"] = dt
        return out

    def can_speculate(self, node_name: str, graph_walk: str) -> bool:
        """May the next loop iteration of this node be launched from the device-resident outputs of the one still
        running (``NodeBatch.speculative``)?"""
        return False

    def prepare_batch(self, batch: NodeBatch) -> PreparedBatch:
        """Per-request input preparation; a request whose preparation raises is failed alone."""
        sub = self.submodules[batch.node_name]
        prepared = PreparedBatch(batch)
        for rid in batch.request_ids:
            try:
                ni = sub.prepare_inputs(batch.graph_walk, batch.fwd_infos[rid], batch.inputs.get(rid, {}))
            except Exception as e:  # noqa: BLE001
                prepared.failed_requests[rid] = f"prepare_inputs failed: {e!r}"
                continue
            prepared.node_inputs.append(ni)
            prepared.request_ids.append(rid)
        return prepared

    def plan(self, prepared: PreparedBatch):
        return prepared

    def execute_forward(self, planned):
        raise NotImplementedError

    def postprocess(self, planned, raw, out: NodeOutput) -> None:
        raise NotImplementedError

    def finalize_batch(self, planned, out: NodeOutput) -> None:
        if self.device.type == "cuda":
            # the device status word travels with the batch: a bounded wait that ran out inside one of its kernels
            # (a late or lost TP / SP peer, a stuck mbarrier) must fail the batch, not stream partial output
            from ..ops import _lib
            if not hasattr(self, "_status_ring"):
                self._status_ring = [torch.zeros(4, dtype=torch.int32).pin_memory() for _ in range(8)]
                self._status_i = 0
            self._status_i = (self._status_i + 1) % len(self._status_ring)
            out.status_host = self._status_ring[self._status_i]
            _lib.status_copy_async(out.status_host)
            io_counters.add_d2h(16)
            ev = torch.cuda.Event()
            ev.record()
            out.completion_event = ev

    def check_batch_status(self, out: NodeOutput) -> str | None:
        """After the batch's completion event: None when every kernel ran to its end, else what gave up (the word is
        cleared so the next batch starts clean). Engines of a TP / SP instance also mark themselves unhealthy: the
        peers' collectives are out of step after a timeout."""
        st = out.status_host
        if st is None:
            return None
        code = int(st[0])
        if code == 0:
            return None
        from ..ops import _lib
        _lib.read_status(clear=True)
        if getattr(self, "tp_group", None) is not None and getattr(self.tp_group, "size", 1) > 1:
            self.unhealthy = True
        return f"device status {code:#x}: {_lib.decode_status(code)} (block {int(st[1])}, aux {int(st[2])}, {int(st[3])})"

    # chunking ---------------------------------------------------------------------------------------
    def execute_with_max_batch_size(self, batch: NodeBatch, max_bs: int) -> NodeOutput:
        if len(batch.request_ids) <= max_bs:
            return self.execute_batch(batch)
        merged = NodeOutput(batch.node_name, batch.graph_walk)
        for i in range(0, len(batch.request_ids), max_bs):
            rids = batch.request_ids[i:i + max_bs]
            part = self.execute_batch(NodeBatch(batch.node_name, batch.graph_walk, rids,
                                                {r: batch.inputs.get(r, {}) for r in rids},
                                                {r: batch.fwd_infos[r] for r in rids}))
            merged.outputs.update(part.outputs)
            merged.stop_loops.update(part.stop_loops)
            merged.failed_requests.update(part.failed_requests)
            merged.allocation_failed |= part.allocation_failed
            merged.allocation_failed_requests += part.allocation_failed_requests
            merged.completion_event = part.completion_event
        return merged

    # lifecycle --------------------------------------------------------------------------------------
    def load_model(self, model, tp_group=None, sp_group=None) -> None:
        for n in self.node_names:
            self.submodules[n] = model.get_submodule(n, self.device, tp_group=tp_group,
                                                     autocast_dtype=model.get_autocast_dtype(), sp_group=sp_group)

    def warmup(self) -> None:
        pass

    def add_request(self, request_id: str, fwd_info) -> None:
        pass

    def remove_request(self, request_id: str) -> None:
        for sub in self.submodules.values():
            sub.cleanup_request(request_id)

    def can_offload(self) -> bool:
        return False

    def offload_request(self, request_id: str) -> int:
        return 0
