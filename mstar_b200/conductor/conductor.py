"""Central per-request state machine. Admits requests (``max_concurrent_requests`` + waiting queue), picks a
replica per node group (least loaded), fans the initial inputs out to the workers that host their consumer nodes,
collects ``WORKER_GRAPHS_DONE`` per walk, asks the model which walk comes next, enforces the output-token budget,
tears requests down on completion / abort / failure, and watches worker heartbeats.

Inside an autoregressive loop the conductor is not involved per token: workers loop locally; only walk
transitions and final outputs come back here.

Reference counterpart: ``Conductor`` (mstar/conductor/conductor.py:209-1227: admission :619-653, ingest :655-785,
replica assignment :475-506, input fan-out :531-576, done processing :909-1063, failure / abort :810-874), request
seeds from md5(request_id) (:53-65). The reference picks replicas at random and has no worker liveness check.
"""
from __future__ import annotations

import logging
import time
from collections import deque
from dataclasses import dataclass, field

from ..graph.ir import GraphEdge
from ..models.base import ForwardPassArgs, WorkerGraph
from ..ops.sampling import request_id_to_seed
from ..utils import ipc_format as ipc
from ..utils.ipc_format import ApiMessageType as AM
from ..utils.ipc_format import ConductorMessageType as CM
from ..utils.ipc_format import Message
from ..utils.ipc_format import WorkerMessageType as WM

log = logging.getLogger("mstar.conductor")


@dataclass
class PartitionState:
    name: str
    walk: str = ""
    pending_graphs: set = field(default_factory=set)
    persist: dict = field(default_factory=dict)
    done: bool = False
    fwd_index: int = 0


@dataclass
class RequestData:
    request_id: str
    body: ipc.NewRequestConductor
    seed: int
    assigned: dict[str, WorkerGraph] = field(default_factory=dict)     # group id -> chosen replica
    partitions: dict[str, PartitionState] = field(default_factory=dict)
    tokens_out: int = 0
    max_tokens: int = 2048
    t_arrive: float = field(default_factory=time.perf_counter)
    t_admit: float = 0.0
    timings: list = field(default_factory=list)


def worker_id_of(rank: int) -> str:
    return f"worker_{rank}"


class Conductor:
    def __init__(self, config: dict, model, comm, *, api_id: str = "api", heartbeat_timeout_s: float = 0.0):
        self.config, self.model, self.comm, self.api_id = config, model, comm, api_id
        self.max_concurrent = int(config.get("max_concurrent_requests", 256))
        self.worker_graphs: list[WorkerGraph] = model.get_worker_graphs(config["node_groups"])
        for wg in self.worker_graphs:
            model.validate_sharding(wg)
        self.walks = model.get_graph_walk_graphs()
        self.kv_nodes = {n for n, t in model.get_node_engine_types().items() if str(getattr(t, "value", t)) == "kv_cache"}
        self.partitions = {p.name: p for p in model.get_partitions()}
        self.requests: dict[str, RequestData] = {}
        self.waiting: deque = deque()
        self.load: dict[str, int] = {wg.graph_id: 0 for wg in self.worker_graphs}
        self.workers_ready: set[str] = set()
        self.all_workers = sorted({worker_id_of(r) for wg in self.worker_graphs for r in wg.ranks})
        self.last_seen: dict[str, float] = {}
        self.heartbeat_timeout_s = heartbeat_timeout_s
        self.dead_workers: set[str] = set()
        self.running = True
        self.stats = dict(admitted=0, completed=0, failed=0, aborted=0)

    # ---- placement helpers ----
    def node_to_workers(self, rd: RequestData | None = None) -> dict[str, list[str]]:
        """node -> worker ids (all ranks of the chosen instance: TP/SP ranks all receive the inputs)."""
        out: dict[str, list[str]] = {}
        for wg in (rd.assigned.values() if rd else self.worker_graphs):
            for n in wg.node_names:
                out.setdefault(n, [])
                for r in wg.ranks:
                    w = worker_id_of(r)
                    if w not in out[n]:
                        out[n].append(w)
        return out

    def _assign(self, rd: RequestData) -> None:
        groups: dict[str, list[WorkerGraph]] = {}
        for wg in self.worker_graphs:
            if any(worker_id_of(r) in self.dead_workers for r in wg.ranks):
                continue
            groups.setdefault(wg.group_id + "|" + ",".join(wg.graph_walks or []), []).append(wg)
        # Replicas are picked least-loaded first, with rank affinity across the request's node groups: once one group
        # of the request sits on some ranks, the other groups prefer their replica on the same ranks (an LLM replica
        # and the codec replica beside it). The request's streaming edges then stay inside one worker process, and a
        # worker's codec batches stay in step with its own decode bursts.
        chosen: set[int] = set()
        for gid, reps in groups.items():
            best = min(reps, key=lambda w: (0 if chosen and chosen & set(w.ranks) else 1, self.load[w.graph_id]))
            rd.assigned[best.graph_id] = best
            self.load[best.graph_id] += 1
            chosen |= set(best.ranks)

    def _graphs_for_walk(self, rd: RequestData, walk: str) -> list[WorkerGraph]:
        nodes = set(self.walks[walk].nodes())
        return [wg for wg in rd.assigned.values() if wg.serves(walk) and nodes & set(wg.node_names)]

    # ---- main loop ----
    def step(self, block_s: float = 0.0) -> bool:
        msgs = self.comm.recv_or_wake(block_s) if block_s > 0 else self.comm.drain()
        for m in msgs:
            try:
                self._handle(m)
            except Exception as e:  # noqa: BLE001
                rid = getattr(m.body, "request_id", None)
                log.exception("conductor: %s failed", m.type)
                if rid:
                    self._fail_requests({rid: f"{type(e).__name__}: {e}"})
        self._try_admit_waiting()
        self._check_heartbeats()
        return bool(msgs)

    def run(self) -> None:
        while self.running:
            self.step(0.01)

    def _handle(self, m: Message) -> None:
        t = m.type
        if t == CM.NEW_REQUEST:
            self.waiting.append(m.body)
        elif t == CM.WORKER_GRAPHS_DONE:
            self._process_worker_graphs_done(m.body)
        elif t == CM.SETUP_DONE:
            self.workers_ready.add(m.body.worker_id)
            self.last_seen[m.body.worker_id] = time.monotonic()
            if set(self.all_workers) <= self.workers_ready:
                self.comm.send(self.api_id, Message(AM.SETUP_DONE, None))
        elif t == CM.HEARTBEAT:
            self.last_seen[m.body.worker_id] = time.monotonic()
        elif t == CM.ABORT_REQUEST:
            self._abort_request(m.body.request_id)
        elif t == CM.FAIL_REQUESTS:
            self._fail_requests(m.body.errors, m.body.status)
        elif t == CM.SHUTDOWN:
            self.shutdown()

    # ---- admission / ingest ----
    def _try_admit_waiting(self) -> None:
        while self.waiting and len(self.requests) < self.max_concurrent:
            body = self.waiting.popleft()
            try:
                self._do_ingest_request(body)
            except Exception as e:  # noqa: BLE001
                log.exception("conductor: ingest of %s failed", body.request_id)
                self.requests.pop(body.request_id, None)
                self.comm.send(self.api_id, Message(AM.REQUEST_FAILED, ipc.RequestFailed(body.request_id, f"{type(e).__name__}: {e}", 400)))

    def _do_ingest_request(self, body: ipc.NewRequestConductor) -> None:
        mk = body.model_kwargs or {}
        seed = int(mk["seed"]) if mk.get("seed") is not None else request_id_to_seed(body.request_id)
        rd = RequestData(body.request_id, body, seed, max_tokens=self.model.get_max_output_tokens(mk))
        rd.t_admit = time.perf_counter()
        self.requests[body.request_id] = rd
        self._assign(rd)
        self.stats["admitted"] += 1
        for pname, pdef in self.partitions.items():
            if pdef.producer_partitions and not pdef.initial_walk:
                continue
            fpa = self.model.get_initial_forward_pass_args(pname, body.initial_input_modalities,
                                                           body.initial_output_modalities, body.initial_signals, mk)
            if fpa is None or not fpa.graph_walk:
                continue
            rd.partitions[pname] = PartitionState(pname)
            self._launch_walk(rd, rd.partitions[pname], fpa)

    def _launch_walk(self, rd: RequestData, ps: PartitionState, fpa: ForwardPassArgs) -> None:
        walk = fpa.graph_walk
        md = fpa.full_metadata
        graphs = self._graphs_for_walk(rd, walk)
        if not graphs:
            raise RuntimeError(f"no worker graph serves walk {walk!r}")
        unplaced = set(self.walks[walk].nodes()) - {n for wg in self.worker_graphs for n in wg.node_names}
        if unplaced:
            raise RuntimeError(f"walk {walk!r} needs nodes that this deployment does not place: {sorted(unplaced)}")
        ps.walk, ps.pending_graphs = walk, {wg.graph_id for wg in graphs}
        ps.fwd_index += 1
        sampling = self.model.resolve_sampling_configs(rd.body.model_kwargs or {})
        sc = {"main": _sampling_dict(sampling.main)}
        sc.update({k: _sampling_dict(v) for k, v in sampling.aux.items()})
        info = ipc.CurrentForwardPassInfo(rd.request_id, walk, bool(md.get("requires_cfg", False)), ps.fwd_index,
                                          rd.seed, int(md.get("max_tokens", rd.max_tokens - rd.tokens_out)), sc,
                                          dict(fpa.step_metadata or {}), {}, ps.name, {},
                                          dict(md.get("dynamic_loop_iter_counts", {})))
        # prefill / decode disaggregation: a KV node that now runs on another worker graph than before takes its
        # pages along (rank i of the new group pulls from rank i of the old one)
        home = rd.__dict__.setdefault("kv_home", {})
        kv_import: dict[str, dict[str, str]] = {}
        for wg in graphs:
            for n in wg.node_names:
                if self.kv_nodes is not None and n in self.kv_nodes and n in self.walks[walk].nodes():
                    old = home.get(n)
                    if old is not None and old.graph_id != wg.graph_id:
                        for src_r, dst_r in zip(old.ranks, wg.ranks):
                            kv_import.setdefault(worker_id_of(dst_r), {})[n] = worker_id_of(src_r)
                    home[n] = wg
        if kv_import:
            info.step_metadata["_kv_import"] = kv_import
        n2w = self.node_to_workers(rd)
        wg2w = {wg.graph_id: [worker_id_of(r) for r in wg.ranks] for wg in rd.assigned.values()}
        per_worker: dict[str, list[GraphEdge]] = {}
        for wg in graphs:
            for r in wg.ranks:
                per_worker.setdefault(worker_id_of(r), [])
        for e in fpa.inputs:
            for w in n2w.get(e.next_node, []):
                if w in per_worker:
                    per_worker[w].append(e)
        for w, edges in per_worker.items():
            gids = [wg.graph_id for wg in graphs if w in wg2w[wg.graph_id]]
            self.comm.send(w, Message(WM.NEW_REQUEST, ipc.NewRequest(rd.request_id, gids, wg2w, edges, info)))
        if fpa.unpersist_tensors:
            for w in {w for ws in wg2w.values() for w in ws}:
                self.comm.send(w, Message(WM.UNPERSIST_TENSORS, ipc.UnpersistTensors(
                    rd.request_id, {u: 1 for u in fpa.unpersist_tensors})))

    # ---- walk completion ----
    def _process_worker_graphs_done(self, b: ipc.WorkerGraphsDone) -> None:
        rd = self.requests.get(b.request_id)
        if rd is None:
            return
        ps = rd.partitions.get(b.partition_name)
        if ps is None or (b.walk and b.walk != ps.walk):
            return
        for k, v in b.persist_signals.items():
            ps.persist.setdefault(k, []).extend(v)
        rd.tokens_out += sum(b.new_token_counts.values())
        rd.timings.append(dict(walk=b.walk, **b.timings))
        ps.pending_graphs -= set(b.worker_graph_ids)
        if ps.pending_graphs:
            return
        self._process_done_forward(rd, ps)

    def _process_done_forward(self, rd: RequestData, ps: PartitionState) -> None:
        md = dict(finished_walk=ps.walk, tokens_out=rd.tokens_out, max_tokens=rd.max_tokens,
                  model_kwargs=rd.body.model_kwargs or {}, output_modalities=rd.body.initial_output_modalities)
        if rd.tokens_out >= rd.max_tokens:
            md["token_budget_exhausted"] = True
        fpa = self.model.get_partition_forward_pass_args(ps.name, md, ps.persist)
        if fpa is None or fpa.request_done or not fpa.graph_walk:
            ps.done = True
            self._send_producer_done(rd, ps.name)
            if all(p.done for p in rd.partitions.values()):
                self._process_request_done(rd)
            return
        self._launch_walk(rd, ps, fpa)

    def _send_producer_done(self, rd: RequestData, partition: str) -> None:
        """Tell the consumers of this partition's streams that no more items will come (final flush)."""
        topo = self.model.get_partition_topology()
        if topo is None:
            return
        n2w = self.node_to_workers(rd)
        for c in topo.outgoing(partition):
            walks = self.partitions[c.to_partition].graph_walks
            consumers = {n for w in walks for n, decl in self.walks[w].nodes().items() if c.edge_name in decl.streaming_inputs}
            for w in {w for n in consumers for w in n2w.get(n, [])}:
                self.comm.send(w, Message(WM.INPUT_SIGNALS, ipc.InputSignals(rd.request_id, [], None, c.to_partition,
                                                                             {c.edge_name})))

    def _process_request_done(self, rd: RequestData) -> None:
        self.stats["completed"] += 1
        prof = dict(queue_s=rd.t_admit - rd.t_arrive, total_s=time.perf_counter() - rd.t_arrive, walks=rd.timings,
                    tokens_out=rd.tokens_out)
        self.comm.send(self.api_id, Message(AM.REQUEST_COMPLETE, ipc.RequestComplete(rd.request_id, {}, prof)))
        self._remove_request(rd.request_id)

    # ---- teardown ----
    def _remove_request(self, request_id: str) -> None:
        rd = self.requests.pop(request_id, None)
        if rd is None:
            return
        for wg in rd.assigned.values():
            self.load[wg.graph_id] = max(0, self.load[wg.graph_id] - 1)
            w = worker_id_of(wg.leader)
            self.comm.send(w, Message(WM.REMOVE_REQUEST, ipc.RemoveRequest(request_id, ipc.MessageSource.CONDUCTOR)))
            for r in wg.ranks[1:]:
                self.comm.send(worker_id_of(r), Message(WM.REMOVE_REQUEST, ipc.RemoveRequest(request_id, ipc.MessageSource.TP_RANK_0)))

    def _abort_request(self, request_id: str) -> None:
        self.waiting = deque(b for b in self.waiting if b.request_id != request_id)
        if request_id in self.requests:
            self.stats["aborted"] += 1
            self._remove_request(request_id)

    def _fail_requests(self, errors: dict[str, str], status: int = 500) -> None:
        for rid, msg in errors.items():
            if rid in self.requests:
                self.stats["failed"] += 1
                self._remove_request(rid)
                self.comm.send(self.api_id, Message(AM.REQUEST_FAILED, ipc.RequestFailed(rid, msg, status)))

    # ---- liveness ----
    def _check_heartbeats(self) -> None:
        if not self.heartbeat_timeout_s:
            return
        now = time.monotonic()
        for w, t in list(self.last_seen.items()):
            if w in self.dead_workers or now - t <= self.heartbeat_timeout_s:
                continue
            self.dead_workers.add(w)
            log.error("conductor: worker %s missed its heartbeat; failing its requests", w)
            victims = {rid: f"worker {w} stopped responding" for rid, rd in self.requests.items()
                       if any(w in [worker_id_of(r) for r in wg.ranks] for wg in rd.assigned.values())}
            self._fail_requests(victims, 503)

    def revive_worker(self, worker_id: str) -> None:
        """A restarted worker (weights reloaded, graphs recaptured) reports SETUP_DONE again and serves new work."""
        self.dead_workers.discard(worker_id)
        self.last_seen[worker_id] = time.monotonic()

    def shutdown(self) -> None:
        self.running = False
        for w in self.all_workers:
            self.comm.send(w, Message(WM.SHUTDOWN, None))


def _sampling_dict(c) -> dict:
    return dict(temperature=c.temperature, top_k=c.top_k, top_p=c.top_p, repetition_penalty=c.repetition_penalty,
                ignore_eos=c.ignore_eos)
