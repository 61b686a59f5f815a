"""Per-GPU worker: owns the engines of the nodes placed on its rank, keeps one ``WalkState`` per (request,
partition), turns arriving signals into ready nodes, lets the micro-scheduler form batches, runs them on a GPU
thread and routes the outputs — to a local node (no copy), to another worker (descriptor over the mesh, data by
peer copy / arena), or to the client through the API server.

Failure handling: a request whose stage fails is failed alone (``FAIL_REQUESTS`` to the conductor); an allocation
failure offloads the request with the most pages to the host pool or holds the batch for a back-off; any other
exception of the main loop fails the requests of the batch in flight and the loop goes on.

Reference counterpart: ``Worker`` (mstar/worker/worker.py:117-2598), ``WorkerGraphsManager``
(mstar/worker/node_manager_utils.py), TP lockstep through ``SCHEDULE_TP`` (:899-923), streaming routing (:660-757),
allocation failure handling (:1252-1300), error containment (:1998-2079).
"""
from __future__ import annotations

import logging
import threading
import os
import time
import traceback
from collections import deque
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field

import torch

from ..communication.communicator import BaseCommunicator
from ..communication.tensors import TensorCommunicationManager
from ..engine.base import NodeBatch, NodeOutput
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, restrict_section
from ..graph.walk_state import WalkState
from ..streaming.stream_buffer import StreamBuffer
from ..utils import ipc_format as ipc
from ..utils.ipc_format import ConductorMessageType as CM
from ..utils.ipc_format import Message
from ..utils.ipc_format import WorkerMessageType as WM
from ..utils.profiler import nvtx_range
from .micro_scheduler import MicroScheduler

log = logging.getLogger("mstar.worker")


@dataclass
class PerRequestInfo:
    request_id: str
    fwd_info: ipc.CurrentForwardPassInfo
    walk_state: WalkState
    worker_graph_ids: list[str]
    worker_graph_to_workers: dict[str, list[str]]
    partition_name: str = "default"
    persist: dict[str, list] = field(default_factory=dict)
    new_token_counts: dict[str, int] = field(default_factory=dict)
    stream_buffers: dict[str, StreamBuffer] = field(default_factory=dict)
    in_flight: int = 0
    remove_pending: bool = False
    kv_wait: set = field(default_factory=set)      # KV nodes whose pages are still on their way from another process
    spec: dict = field(default_factory=dict)       # node -> ids of the speculative flights that run its NEXT iterations
    spec_marked: set = field(default_factory=set)  # nodes marked running on behalf of such a flight
    stream_targets: dict = field(default_factory=dict)   # streaming edge name -> node of this walk that consumes it
    t_start: float = field(default_factory=time.perf_counter)
    timings: dict = field(default_factory=dict)


@dataclass
class _Flight:
    """One batch between its launch and the read-back of its results."""
    fid: int
    batch: NodeBatch
    engine: object
    fut: object = None                 # future of the launch (GPU work being queued on the launch thread)
    pending: object = None             # PendingBatch once the launch returned
    error: BaseException | None = None
    speculative: bool = False
    chain: int = 0                     # speculative launches in a row that led to this one
    spec_tried: bool = False
    t_submit: float = 0.0


class Worker:
    def __init__(self, worker_id: str, rank: int, model, node_names: list[str], comm: BaseCommunicator,
                 tensors: TensorCommunicationManager, engine_manager, *, node_to_workers: dict[str, list[str]],
                 conductor_id: str = "conductor", api_id: str = "api", tp_followers: list[str] | None = None,
                 is_tp_follower: bool = False, max_batch_size: int = 64, async_gpu: bool = True,
                 heartbeat_s: float = 0.0, log_stats: bool = False, publish_persisted: bool = True,
                 node_walks: dict[str, set | None] | None = None, parallel_nodes: set | None = None,
                 instance_workers: set | None = None):
        self.worker_id, self.rank, self.model = worker_id, rank, model
        # nodes that run on every rank of this worker's tensor- / sequence-parallel instance in lockstep, and the
        # workers of that instance. Every rank keeps such a node's outputs for itself; what leaves the instance
        # (client, nodes elsewhere, the conductor) is sent by the instance's first rank only.
        self.parallel_nodes = set(parallel_nodes) if parallel_nodes is not None else None
        self.instance_workers = set(instance_workers or ())
        # node -> the walks in which this worker runs it (None / absent: every walk). A node placed per walk (prompt
        # passes here, decoding elsewhere) must stay out of the other walks even when the walk reaches this worker
        # for another of its nodes.
        self.node_walks = dict(node_walks or {})
        # per-request profile (node timings, tensor transfers), collected only when the server logs request statistics
        self.profile = None
        if log_stats or os.environ.get("MSTAR_LOG_STATS"):
            from ..profile.records import WorkerProfile
            self.profile = WorkerProfile(worker_id)
            tensors.log_transfers = True
        self.node_names = set(node_names)
        self.comm, self.tensors, self.engines = comm, tensors, engine_manager
        self.node_to_workers = node_to_workers
        self.conductor_id, self.api_id = conductor_id, api_id
        self.tp_followers = tp_followers or []
        self.is_tp_follower = is_tp_follower
        self.scheduler = MicroScheduler(max_batch_size=max_batch_size, is_tp_follower=is_tp_follower)
        self.scheduler.follow_nodes = self.parallel_nodes
        self.scheduler.limit_fn = self._node_batch_limit
        self.scheduler.defer_fn = self._defer_batch
        # batch gathering: a batch is held back for a moment while requests that would join it are still on the GPU in
        # this worker (their next input is about to exist) or while new requests are still arriving in a burst;
        # without it two groups of streams that got out of step keep alternating as two half batches for ever
        self._gather_running_s = float(os.environ.get("MSTAR_GATHER_RUNNING_MS", "60")) / 1e3
        self._gather_arrival_s = float(os.environ.get("MSTAR_GATHER_ARRIVAL_MS", "4")) / 1e3
        self._last_arrival = 0.0
        self._by_walk_node: dict[tuple[str, str], dict] = {}       # (node, walk) -> live request states that run it
        self.trace = [] if os.environ.get("MSTAR_TRACE_WORKER") else None
        # persisted tensors (a prefill's last token, ...) come back through the conductor in a later walk. They only
        # need to be published for other processes when some node is split over node groups by walk (prefill and
        # decode on different workers); otherwise the request stays on this worker and the store lookup is local
        self._publish_persisted = publish_persisted
        self._stall_log_s = float(os.environ.get("MSTAR_STALL_LOG_S", "15"))
        self._last_stall_scan, self._stall_logged = time.monotonic(), set()
        self._deferred_stream_end: dict[tuple[str, str], list] = {}    # stream ends waiting for this rank's own producer
        self._deferred_new: dict[tuple[str, str], list] = {}   # NEW_REQUEST of a walk whose predecessor is still in flight here
        self._done_queue: list | None = None      # walk-completion messages held back while a batch is being finished
        self._emit_buf: list | None = None        # client-bound outputs of the batch being finished, sent as one message
        self.walks = model.get_graph_walk_graphs()
        self.topology = model.get_partition_topology()
        self.requests: dict[tuple[str, str], PerRequestInfo] = {}     # (request_id, partition) -> info
        self.running = True
        # Execution pipeline. Launches (input preparation, planning, kernel / graph launches, queued result copies)
        # run on ONE launch thread, so the CUDA stream sees them in submission order and never waits for the host;
        # the main loop polls each flight's event and reads results back only when they are there. Every engine has
        # its own queue of flights: while the decode burst N of a KV engine runs, burst N+1 is already queued behind
        # it (speculation: its inputs are the ids that burst N leaves on the device), and codec / encoder batches of
        # other engines are queued as soon as their inputs exist. The GPU goes from one batch to the next without
        # waiting for scheduling, routing or bookkeeping.
        self.gpu_thread = ThreadPoolExecutor(1, thread_name_prefix=f"{worker_id}-gpu",
                                             initializer=self._bind_device) if async_gpu else None
        self._pipes: dict[int, deque] = {}           # id(engine) -> flights in launch order
        self._next_fid = 0
        lockstep = bool(is_tp_follower or tp_followers)
        self._spec_enabled = bool(async_gpu and not lockstep and os.environ.get("MSTAR_SPECULATE", "1") != "0")
        self._max_chain = int(os.environ.get("MSTAR_MAX_CONSECUTIVE_SPEC_STEPS", "1024"))
        # flights of one engine that may be queued at once: the running batch plus this many speculative
        # continuations (2: the GPU still has a queued batch while the host digests the results of the one that
        # just finished, which takes about as long as a burst runs)
        self._spec_depth = max(1, int(os.environ.get("MSTAR_SPEC_DEPTH", "2")))
        # every engine launches on its own CUDA stream when the worker hosts several (MSTAR_ENGINE_STREAMS=0: one
        # stream): a codec batch then does not queue behind the decode bursts that were launched ahead of it.
        # Stateless engines (codecs, encoders) get the higher priority: their batches are short and sit on the
        # latency path of a stream's next chunk. Outputs only change engines after their flight was read back, so
        # no cross-stream waits are needed; device inputs are recorded on the consuming stream for the allocator.
        n_eng = len(getattr(engine_manager, "engines", []) or [])
        self._engine_streams = (os.environ.get("MSTAR_ENGINE_STREAMS", "1") != "0") and n_eng > 1 and not lockstep
        self._streams: dict[int, object] = {}        # id(engine) -> CUDA stream
        self.spec_stats = dict(launched=0, discarded_rows=0, cancelled=0)
        self.heartbeat_s = heartbeat_s
        self._last_beat = time.monotonic()
        self.phase_times: dict[str, list[float]] = {}
        self.iterations = 0
        self._streaming_requests: set[tuple[str, str]] = set()      # request states that own stream buffers
        # ... and those of them whose buffers or consumer nodes changed since they were last looked at: only these
        # are polled (new items, producer done, consumer node finished an iteration, another input arrived)
        self._stream_dirty: set[tuple[str, str]] = set()
        # host time by phase of the main loop (seconds): where a step's latency goes when the GPU is not the limit
        self.phase_s = dict(wait=0.0, messages=0.0, streams=0.0, finish=0.0, build=0.0, execute=0.0)
        self.batches_by_node: dict[str, list] = {}
        self._kv_early: dict[tuple[str, str], ipc.KVImport] = {}     # KV_IMPORT that overtook its NEW_REQUEST

    # ------------------------------------------------------------------ messages
    def _process_messages(self, msgs: list[Message]) -> None:
        for m in msgs:
            try:
                t = m.type
                if t == WM.NEW_REQUEST:
                    self._on_new_request(m.body)
                elif t == WM.INPUT_SIGNALS:
                    self._on_input_signals(m.body)
                elif t == WM.REMOVE_REQUEST:
                    self._on_remove_request(m.body)
                elif t == WM.STOP_LOOPS:
                    self._on_stop_loops(m.body)
                elif t == WM.SCHEDULE_TP:
                    self.scheduler.push_tp_decision(m.body.node_name, m.body.graph_walk, m.body.request_ids)
                elif t == WM.UNPERSIST_TENSORS:
                    for u, n in m.body.uuid_to_ref_count.items():
                        self.tensors.store.unpersist(u)
                elif t == WM.TENSOR_RECEIVED:
                    for u, n in m.body.successful_tensors.items():
                        self.tensors.dereference(m.body.request_id, u, n)
                elif t == WM.TENSOR_RECEIVED_BATCH:
                    for r in m.body.items:
                        for u, n in r.successful_tensors.items():
                            self.tensors.dereference(r.request_id, u, n)
                elif t == WM.KV_EXPORT:
                    self._on_kv_export(m.body)
                elif t == WM.KV_IMPORT:
                    self._on_kv_import(m.body)
                elif t == WM.SHUTDOWN:
                    self.running = False
            except Exception as e:  # noqa: BLE001
                rid = getattr(m.body, "request_id", None)
                log.exception("worker %s: message %s failed", self.worker_id, m.type)
                if rid:
                    self._fail_requests({rid: f"{type(e).__name__}: {e}"})

    def _node_batch_limit(self, node: str, walk: str) -> int:
        """Largest batch the node's submodule takes for this walk (1 for nodes that run one request at a time)."""
        try:
            sub = self.engines.engine_for(node).submodules[node]
            return int(sub.max_batch_size(walk)) if sub.can_batch(walk) else 1
        except Exception:  # noqa: BLE001
            return 1 << 30

    def _defer_batch(self, node: str, walk: str, rids: list, waited_s: float) -> bool:
        """Hold this batch back? Yes while (a) requests are still arriving in a burst (a few milliseconds), or (b)
        other live requests of the same walk will need this node too and are on the GPU right now, in this node or in
        the node that feeds it (bounded by the gather window)."""
        now = time.monotonic()
        if waited_s < self._gather_arrival_s and now - self._last_arrival < 0.0015:
            return True
        if waited_s >= self._gather_running_s:
            return False
        have = set(rids)
        for (rid, part), pri in self.requests.items():
            if pri.in_flight <= 0 or pri.fwd_info.graph_walk != walk or f"{rid}|{part}" in have:
                continue
            st = pri.walk_state.nodes.get(node)
            if st is not None and not st.scope.done and (st.running or not st.done):
                return True
        if self.topology is not None and self._streaming_requests:
            # stream consumers: their producers run in another partition's request state of the same request
            for (rid, part) in self._streaming_requests:
                if f"{rid}|{part}" in have:
                    continue
                pri = self.requests.get((rid, part))
                if pri is None or pri.fwd_info.graph_walk != walk or node not in pri.walk_state.nodes:
                    continue
                if pri.walk_state.nodes[node].scope.done:
                    continue
                for c in self.topology.incoming(part):
                    src = self.requests.get((rid, c.from_partition))
                    if src is not None and src.in_flight > 0:
                        return True
        return False

    def _section_for(self, walk: str):
        sec = self.walks.get(walk)
        if sec is None:
            raise KeyError(f"unknown graph walk {walk!r}")
        mine = {n for n in self.node_names if self.node_walks.get(n) is None or walk in self.node_walks[n]}
        return restrict_section(sec, mine)

    def _on_new_request(self, b: ipc.NewRequest) -> None:
        info = b.request_info
        sec = self._section_for(info.graph_walk)
        if sec is None:
            return
        prev = self.requests.get((b.request_id, info.partition_name))
        if prev is not None and prev.in_flight > 0 and prev.fwd_info.graph_walk != info.graph_walk:
            # the previous walk's last batch has not been read back on THIS rank yet (a rank of a parallel instance
            # can trail the rank that reported the walk's end): the new walk starts when it has, or that batch's
            # completion would be booked on the new walk's state
            self._deferred_new.setdefault((b.request_id, info.partition_name), []).append(b)
            return
        # read, not popped: workers of an in-process deployment receive the same message object
        imports = (info.step_metadata or {}).get("_kv_import", {}).get(self.worker_id, {})
        remote_kv: set[str] = set()
        for node, src_worker in imports.items():
            if node in self.node_names and (self.node_walks.get(node) is None or info.graph_walk in self.node_walks[node]):
                from .engine_manager import lookup_kv_engine
                src = lookup_kv_engine(src_worker, node)
                if src is None:
                    # the pool that ran the prefill lives in another process: ask its worker for the pages and keep
                    # the node unscheduled until they are in this pool
                    remote_kv.add(node)
                    self.comm.send(src_worker, Message(WM.KV_EXPORT, ipc.KVExport(b.request_id, node, self.worker_id)))
                    continue
                self.engines.engine_for(node).import_kv_from(src, b.request_id, info)
        key = (b.request_id, info.partition_name)
        old = self.requests.get(key)
        ws = WalkState(sec, b.request_id, on_release=lambda e, rid=b.request_id: self._release_edge(rid, e))
        for loop_name, iters in (info.dynamic_loop_iter_counts or {}).items():
            sc = ws.scopes.get(loop_name)
            if sc is not None:
                sc.loop = _with_max_iters(sc.loop, int(iters))
        pri = PerRequestInfo(b.request_id, info, ws, b.partition_worker_graph_ids, b.worker_graph_to_workers,
                             info.partition_name)
        if old is not None:
            pri.stream_buffers = old.stream_buffers
            pri.persist = old.persist
        pri.kv_wait = remote_kv
        self.requests[key] = pri
        self._last_arrival = time.monotonic()
        if self.trace is not None:
            self.trace.append((time.monotonic(), "new_request", info.graph_walk, b.request_id))
        self._setup_streams(pri)
        for e in b.initial_inputs:
            self._ingest(pri, e)
        self._refresh_ready(pri)
        for node in list(remote_kv):
            early = self._kv_early.pop((b.request_id, node), None)
            if early is not None:
                self._on_kv_import(early)

    def _setup_streams(self, pri: PerRequestInfo) -> None:
        if self.topology is None:
            return
        for c in self.topology.incoming(pri.partition_name):
            if c.edge_name not in pri.stream_buffers:
                pri.stream_buffers[c.edge_name] = StreamBuffer(pri.request_id, c.edge_name, c.from_partition,
                                                               c.chunk_policy_factory())
        if pri.stream_buffers:
            self._streaming_requests.add((pri.request_id, pri.partition_name))
            self._stream_dirty.add((pri.request_id, pri.partition_name))

    def _on_input_signals(self, b: ipc.InputSignals) -> None:
        pri = self.requests.get((b.request_id, b.partition_name))
        if pri is None:
            # normal for stream edges towards a partition the request does not use (text-only output of an omni model)
            log.debug("worker %s: inputs %s for a request it does not hold (%s, partition %s)", self.worker_id,
                      [e.name for e in b.inputs], b.request_id, b.partition_name)
            return
        if b.request_info is not None and b.request_info.graph_walk != pri.fwd_info.graph_walk:
            pri.fwd_info = b.request_info
        for name in b.producer_done or ():
            sb = pri.stream_buffers.get(name)
            if sb is None:
                continue
            if self.is_tp_follower and self.topology is not None:
                # the end of a stream is announced when the producing instance's FIRST rank has finished; a rank that
                # follows that instance and feeds this consumer from its own copy may still have the last items in
                # flight: the end then takes effect when this rank's own producer walk is done
                src = next((self.requests.get((b.request_id, c.from_partition))
                            for c in self.topology.incoming(b.partition_name) if c.edge_name == name), None)
                if src is not None and (src.in_flight > 0 or not src.walk_state.done):
                    self._deferred_stream_end.setdefault((b.request_id, src.partition_name), []).append(
                        (b.partition_name, name))
                    continue
            sb.signal_done()
            self._stream_dirty.add((b.request_id, b.partition_name))
        for e in b.inputs:
            self._ingest(pri, e)
        self._refresh_ready(pri)

    def _ingest(self, pri: PerRequestInfo, e: GraphEdge) -> None:
        sb = pri.stream_buffers.get(e.name) if e.is_streaming else None
        if pri.stream_buffers:
            self._stream_dirty.add((pri.request_id, pri.partition_name))
        if sb is not None:
            for ti in e.tensor_info:
                t = self.tensors.read(ti)
                if isinstance(t, torch.Tensor) and t.dim() == 1 and t.numel() > 1 and not t.is_floating_point():
                    for i, v in enumerate(t.tolist()):      # a burst of token ids in one tensor: plain ints
                        sb.put(f"{ti.uuid}:{i}", v)
                else:
                    sb.put(ti.uuid, t)
            return
        pri.walk_state.ingest(e)

    def _poll_stream_buffers(self) -> None:
        if not self._stream_dirty:
            return
        dirty, self._stream_dirty = self._stream_dirty, set()
        for key in dirty:
            pri = self.requests.get(key)
            if pri is None:
                self._streaming_requests.discard(key)
                continue
            nodes = pri.walk_state.nodes
            for name, sb in pri.stream_buffers.items():
                target = pri.stream_targets.get(name)
                if target is None:
                    target = next((n for n, st in nodes.items() if name in st.decl.streaming_inputs), "")
                    pri.stream_targets[name] = target
                st = nodes.get(target)
                if st is None or name in st.cur or st.running or st.done or not sb.has_chunk_ready():
                    continue
                if not st.is_ready_for_streaming():
                    continue
                chunk = sb.pop_chunk()
                data = chunk.data["data"]
                if isinstance(data, torch.Tensor):
                    t = data
                elif isinstance(data, list) and data:
                    if isinstance(data[0], torch.Tensor):
                        t = torch.cat([d.reshape(-1) for d in data])
                    else:
                        t = torch.tensor(data, dtype=torch.int64)
                else:
                    t = torch.zeros(0, dtype=torch.int64)
                ti = self.tensors.store_and_return_tensor_info(pri.request_id, t)
                edge = GraphEdge(target, name, [ti], is_streaming=True, final_stream_chunk=chunk.is_final)
                pri.walk_state.ingest(edge)
                pri.fwd_info.step_metadata = dict(pri.fwd_info.step_metadata or {}, chunk_index=chunk.chunk_index,
                                                  chunk_start=chunk.start_offset, final_chunk=chunk.is_final)
                self._refresh_ready(pri)

    def _refresh_ready(self, pri: PerRequestInfo) -> None:
        for n in pri.walk_state.ready_nodes(allow_streaming=False):
            if n in pri.kv_wait:
                continue
            self.scheduler.mark_ready(n, pri.fwd_info.graph_walk, _rk(pri))

    # ------------------------------------------------------------------ KV hand-off between processes
    def _on_kv_export(self, b: ipc.KVExport) -> None:
        """Prefill side: pack the request's pages and hand the descriptors to the worker that asked."""
        eng = self.engines.engine_for(b.node_name)
        meta, tensors = eng.export_kv(b.request_id)
        infos = {}
        for name, t in tensors.items():
            ti = self.tensors.store_and_return_tensor_info(b.request_id, t)
            infos[name] = self.tensors.prepare_for_remote(ti, b.reply_to)
        self.comm.send(b.reply_to, Message(WM.KV_IMPORT, ipc.KVImport(b.request_id, b.node_name, self.worker_id, meta, infos)))

    def _on_kv_import(self, b: ipc.KVImport) -> None:
        """Decode side: store the pages, acknowledge the tensors, release the node."""
        pris = [p for (rid, _), p in self.requests.items() if rid == b.request_id and b.node_name in p.kv_wait]
        if not pris:
            self._kv_early[(b.request_id, b.node_name)] = b      # the NEW_REQUEST is still on its way
            return
        pri = pris[0]
        tensors = {name: self.tensors.read(ti, self.tensors.device) for name, ti in b.tensor_info.items()}
        self.engines.engine_for(b.node_name).import_kv(b.request_id, pri.fwd_info, b.meta, tensors)
        if b.tensor_info:
            self.comm.send(b.source_worker, Message(WM.TENSOR_RECEIVED, ipc.TensorReceived(
                b.request_id, {ti.uuid: 1 for ti in b.tensor_info.values()})))
        for p in pris:
            p.kv_wait.discard(b.node_name)
            self._refresh_ready(p)

    def _on_remove_request(self, b: ipc.RemoveRequest) -> None:
        for key in [k for k in self.requests if k[0] == b.request_id]:
            pri = self.requests[key]
            if pri.in_flight:
                pri.remove_pending = True       # deferred: a batch with this request is on the GPU
                continue
            self._drop(key)
        if b.source == ipc.MessageSource.CONDUCTOR:
            for f in self.tp_followers:
                self.comm.send(f, Message(WM.REMOVE_REQUEST, ipc.RemoveRequest(b.request_id, ipc.MessageSource.TP_RANK_0)))

    def _drop(self, key) -> None:
        pri = self.requests.pop(key, None)
        if pri is None:
            return
        self.scheduler.remove_request(_rk(pri))
        pri.walk_state.clear()
        self._deferred_new.pop(key, None)
        self._deferred_stream_end.pop(key, None)
        self._stall_logged.discard(key)
        if not any(k[0] == key[0] for k in self.requests):
            self.engines.remove_request(key[0])
            self.tensors.remove_request(key[0])
            if self.profile is not None:
                self.profile.drop(key[0])

    def _on_stop_loops(self, b: ipc.StopLoops) -> None:
        pri = self.requests.get((b.request_id, b.partition_name))
        if pri is not None:
            for ln in b.loop_names:
                pri.walk_state.stop_loop(ln)

    def _release_edge(self, request_id: str, e: GraphEdge) -> None:
        for ti in e.tensor_info:
            if ti.source_entity == self.worker_id:
                self.tensors.dereference(request_id, ti.uuid)

    # ------------------------------------------------------------------ batches
    def _build_node_batch(self, node: str, walk: str, rkeys: list[str]) -> NodeBatch | None:
        inputs, infos, rids = {}, {}, []
        for rk in rkeys:
            rid, part = rk.split("|", 1)
            pri = self.requests.get((rid, part))
            if pri is None:
                continue
            ins = {}
            for name, edge in pri.walk_state.inputs_of(node).items():
                ins[name] = [self._read_input(rid, name, ti) for ti in edge.tensor_info]
            sc = pri.walk_state.nodes[node].scope
            if sc.loop is not None:          # iterations the node may still run (bound of a decode burst)
                pri.fwd_info.step_metadata = dict(pri.fwd_info.step_metadata or {},
                                                  _loop_remaining=max(1, sc.loop.max_iters - sc.curr_iter))
            pri.walk_state.mark_running(node)
            pri.in_flight += 1
            inputs[rid] = ins
            infos[rid] = pri.fwd_info
            rids.append(rid)
        if not rids:
            return None
        b = NodeBatch(node, walk, rids, inputs, infos)
        b.partitions = {rk.split("|", 1)[0]: rk.split("|", 1)[1] for rk in rkeys}
        return b

    def _bind_device(self) -> None:
        """The CUDA current device is a per-thread setting and new threads start on device 0: bind the launch thread
        to this worker's GPU (kernel launches through the C ABI use the thread's current device and stream)."""
        dev = next((e.device for e in getattr(self.engines, "engines", []) if e.device.type == "cuda"), None)
        if dev is not None:
            torch.cuda.set_device(dev)

    def _launch(self, fl: _Flight):
        """Launch thread: queue the batch's GPU work; returns the engine's PendingBatch without waiting for it."""
        eng, batch = fl.engine, fl.batch
        with nvtx_range(f"{batch.node_name}:{batch.graph_walk}:{len(batch.request_ids)}"):
            t0 = time.perf_counter()
            if self._engine_streams and eng.device.type == "cuda":
                st = self._streams.get(id(eng))
                if st is None:
                    prio = 0 if hasattr(eng, "cache") else -1
                    if self.tp_followers or self.is_tp_follower:
                        # a tensor- / sequence-parallel instance runs in lockstep: its kernels wait (bounded) for the
                        # peers', so on this rank nothing may hold them back. The instance's engine gets the high
                        # priority here and the other engines of the rank (a VAE decode of seconds) the low one.
                        prio = -1 if hasattr(eng, "cache") else 0      # the sharded model sits on the KV-cache engine
                    st = self._streams[id(eng)] = torch.cuda.Stream(device=eng.device, priority=prio)
                for ins in batch.inputs.values():
                    for ts in ins.values():
                        for t in ts:
                            if isinstance(t, torch.Tensor) and t.is_cuda:
                                t.record_stream(st)
                with torch.cuda.stream(st):
                    pend = eng.launch_batch(batch)
            else:
                pend = eng.launch_batch(batch)
            self.phase_s["execute"] += time.perf_counter() - t0
        return pend

    def _postprocess_batch(self, batch: NodeBatch, out: NodeOutput, fl: _Flight | None = None) -> None:
        if out.completion_event is not None:
            out.completion_event.synchronize()
        spec = fl is not None and fl.speculative
        bad = self.engines.engine_for(batch.node_name).check_batch_status(out)
        if bad is not None:
            # a kernel of this batch left through its timeout exit: its output is partial, fail every request of it
            log.error("worker %s: %s:%s %s", self.worker_id, batch.node_name, batch.graph_walk, bad)
            out.failed_requests = {rid: bad for rid in batch.request_ids}
            out.allocation_failed = False
        if out.allocation_failed:
            if spec:
                self._cancel_speculation(fl)        # nothing was launched: the loop goes on through the scheduler
            else:
                self._handle_allocation_failure(batch, out)
            return
        if out.failed_requests:
            self._fail_requests(out.failed_requests)
        node = batch.node_name
        for rid in batch.request_ids:
            pri = self.requests.get((rid, batch.partitions[rid]))
            if pri is None:
                continue
            pri.in_flight -= 1
            if spec:
                if fl.fid not in pri.spec.get(node, ()):
                    # the loop ended (stop token, budget, abort) in an iteration before: this row's work is dropped
                    self.spec_stats["discarded_rows"] += 1
                    if pri.remove_pending and pri.in_flight == 0:
                        self._drop((rid, pri.partition_name))
                    self._start_deferred_walk(rid, pri)
                    continue
                pri.spec[node].remove(fl.fid)
                pri.spec_marked.discard(node)
            if rid in out.failed_requests:
                continue
            try:
                self._complete_node(pri, batch, out.outputs.get(rid, {}), out.stop_loops.get(rid, set()),
                                    out.iterations.get(rid, 1))
            except Exception as e:  # noqa: BLE001
                log.exception("worker %s: routing outputs of %s failed", self.worker_id, rid)
                self._fail_requests({rid: f"{type(e).__name__}: {e}"})
            if pri.remove_pending and pri.in_flight == 0:
                self._drop((rid, pri.partition_name))
            self._start_deferred_walk(rid, pri)

    def _log_stalled_requests(self) -> None:
        """Diagnostic: requests that hold a walk here, have nothing on the device and no node ready, logged once with
        what every unfinished node still misses (an input that was routed elsewhere, a walk that never got its
        first edge)."""
        for key, pri in self.requests.items():
            ws = pri.walk_state
            if pri.in_flight or ws.done or key in self._stall_logged or time.perf_counter() - pri.t_start < self._stall_log_s:
                continue
            ready = ws.ready_nodes(allow_streaming=False)
            if ready:
                self._stall_logged.add(key)
                log.warning("worker %s: request %s idle in walk %s for %.0f s with nodes ready but not running: %s "
                            "(waiting for pages of another pool: %s; scheduler queue: %s; leader decisions pending: %d)",
                            self.worker_id, key[0], pri.fwd_info.graph_walk, time.perf_counter() - pri.t_start, ready,
                            sorted(pri.kv_wait), {k: list(v) for k, v in self.scheduler.ready.items() if v},
                            len(self.scheduler._tp_queue))
                continue
            if ws.ready_nodes(allow_streaming=True):
                continue
            waiting = {n: sorted(st.missing()) for n, st in ws.nodes.items()
                       if not st.done and not st.running and not st.scope.done}
            if waiting:
                self._stall_logged.add(key)
                log.warning("worker %s: request %s idle in walk %s for %.0f s; nodes waiting for inputs: %s",
                            self.worker_id, key[0], pri.fwd_info.graph_walk, time.perf_counter() - pri.t_start, waiting)

    def _start_deferred_walk(self, rid: str, pri: PerRequestInfo) -> None:
        if pri.in_flight == 0 and self._deferred_new:
            for nb in self._deferred_new.pop((rid, pri.partition_name), []):
                self._on_new_request(nb)

    def _complete_node(self, pri: PerRequestInfo, batch: NodeBatch, tensors: dict, stops: set,
                       iterations: int = 1) -> None:
        ws = pri.walk_state
        node = batch.node_name
        for ln in stops:
            ws.stop_loop(ln)
        if stops:
            self._broadcast_stops(pri, stops)
        decl = ws.nodes[node].decl
        edges = []
        for e in decl.outputs:
            t = tensors.get(e.name)
            if t is None:
                continue
            ne = e.clone(with_tensors=False)
            refs = sum(1 for o in decl.outputs if o.name == e.name)
            if not isinstance(t, (list, tuple)):
                t = [t]
            # tensors on their way to the client outlive the request's teardown: they are released by the API
            # server's TENSOR_RECEIVED acknowledgement, not by REMOVE_REQUEST
            owner = pri.request_id + "#emit" if e.next_node == EMIT_TO_CLIENT else pri.request_id
            ne.tensor_info = [self.tensors.store_and_return_tensor_info(owner, x, refs=refs, persist=e.persist)
                              for x in t if isinstance(x, torch.Tensor)]
            edges.append(ne)
            if e.conductor_new_token and not (self.is_tp_follower and self.instance_workers and
                                              (self.parallel_nodes is None or node in self.parallel_nodes)):
                pri.new_token_counts[e.name] = pri.new_token_counts.get(e.name, 0) + max(1, iterations)
        comp = ws.complete(node, edges, iterations=iterations)
        if pri.stream_buffers:
            self._stream_dirty.add((pri.request_id, pri.partition_name))
        if pri.spec.get(node):
            st = ws.nodes[node]
            if ws.done or st.scope.done or st.done or not st.is_ready():
                # the loop ended with this iteration: whatever the speculative launches compute for this request is
                # dropped when those flights are read back
                pri.spec[node] = []
                ws.rollback_speculation(node)
            else:
                ws.mark_running(node)       # iteration N+1 is already queued on the GPU, fed from the device
                pri.spec_marked.add(node)
        self._send_outputs(pri, comp.route, producer=node)
        if self.instance_workers and self.parallel_nodes and node not in self.parallel_nodes:
            # a node of this rank alone (an encoder) fed a node that runs on every rank of the instance: the local
            # hand-over reached this rank only, the other ranks get the edge as a message
            peers = [e for e in comp.delivered if e.next_node in self.parallel_nodes]
            if peers:
                self._send_outputs(pri, peers, producer=node, skip_self=True)
        self._refresh_ready(pri)
        if comp.walk_done:
            self._walk_done(pri)

    def _send_outputs(self, pri: PerRequestInfo, edges: list[GraphEdge], producer: str | None = None,
                      skip_self: bool = False) -> None:
        by_worker: dict[str, list[GraphEdge]] = {}
        # the producer ran on every rank of a parallel instance: each rank feeds itself, the first rank speaks for all
        lockstep = bool(self.instance_workers) and producer is not None and \
            (self.parallel_nodes is None or producer in self.parallel_nodes)
        for e in edges:
            if skip_self:           # already handed over and booked on this rank: only the other workers of the node
                for w in self.node_to_workers.get(e.next_node, []):
                    if w != self.worker_id:
                        by_worker.setdefault(w, []).append(e)
                continue
            if e.persist and lockstep and self.is_tp_follower:
                pass        # the instance's first rank reports (and publishes) its copy
            elif e.persist:
                # a persisted tensor can be handed by the conductor to ANY worker in a later walk (prefill / decode
                # split): when some worker lives in another process, publish it now (arena block or CUDA IPC handle),
                # since only the owner can do that
                peers = {w for ws_ in self.node_to_workers.values() for w in ws_} if self._publish_persisted else ()
                if any(not self.tensors.is_local(w) for w in peers):
                    e.tensor_info = [self.tensors.prepare_for_remote(ti, "*") for ti in e.tensor_info]
                pri.persist.setdefault(e.name, []).extend(e.tensor_info)
            if e.next_node == EMPTY_DESTINATION:
                continue
            if e.next_node == EMIT_TO_CLIENT:
                if lockstep and self.is_tp_follower:
                    continue
                emit_owner = pri.request_id + "#emit"
                for ti in e.tensor_info:        # a loop's last output was stored as an intermediate: re-own it
                    if self.tensors.store.owner_of(ti.uuid) not in (None, emit_owner):
                        self.tensors.store.adopt(ti.uuid, emit_owner)
                infos = [self._publish(pri.request_id, e.name, ti, self.api_id) for ti in e.tensor_info]
                rt = ipc.ResultTensors(pri.request_id, e.output_modality or "text", infos,
                                       {"name": e.name, "partition": pri.partition_name}, self.worker_id)
                if self._emit_buf is not None:      # inside a batch's read-back: one message for all its requests
                    self._emit_buf.append(rt)
                else:
                    self.comm.send(self.api_id, Message(ipc.ApiMessageType.RESULT_TENSORS, rt))
                continue
            for w in self.node_to_workers.get(e.next_node, []):
                if lockstep and w != self.worker_id and (w in self.instance_workers or self.is_tp_follower):
                    continue
                by_worker.setdefault(w, []).append(e)
        for w, es in by_worker.items():
            # edges of a streaming connection belong to the CONSUMER partition's request state, also when producer
            # and consumer partitions share this worker (colocated placements)
            groups: dict[str, list[GraphEdge]] = {}
            for e in es:
                part = pri.partition_name
                if self.topology is not None:
                    for c in self.topology.outgoing(pri.partition_name):
                        if e.name == c.edge_name:
                            part = c.to_partition
                groups.setdefault(part, []).append(e)
            for part, ges in groups.items():
                if w == self.worker_id:
                    target = self.requests.get((pri.request_id, part))
                    if target is not None:
                        for e in ges:
                            self._ingest(target, e)
                        self._refresh_ready(target)
                    else:       # the consumer partition's NEW_REQUEST has not arrived yet: deliver through the mailbox
                        self.comm.send(w, Message(WM.INPUT_SIGNALS, ipc.InputSignals(pri.request_id, ges, None, part)))
                    continue
                out_edges = []
                for e in ges:
                    c = e.clone(with_tensors=False)
                    c.tensor_info = [self._publish(pri.request_id, e.name, ti, w) for ti in e.tensor_info]
                    out_edges.append(c)
                self.comm.send(w, Message(WM.INPUT_SIGNALS, ipc.InputSignals(pri.request_id, out_edges, None, part)))

    def _publish(self, request_id: str, edge: str, ti, dst: str):
        """Make a tensor readable by ``dst`` (arena block / IPC handle when it lives in another process); the copy is
        charged to the request's profile when statistics are on."""
        if self.profile is None or self.tensors.is_local(dst):
            return self.tensors.prepare_for_remote(ti, dst)
        t0 = time.perf_counter()
        out = self.tensors.prepare_for_remote(ti, dst)
        self.profile.record_transfer(request_id, "tx", edge, self.worker_id, dst, ti.nbytes, time.perf_counter() - t0)
        return out

    def _read_input(self, request_id: str, edge: str, ti):
        if self.profile is None or self.tensors.is_local(ti.source_entity):
            return self.tensors.read(ti)
        t0 = time.perf_counter()
        t = self.tensors.read(ti)
        self.profile.record_transfer(request_id, "rx", edge, ti.source_entity, self.worker_id, ti.nbytes,
                                     time.perf_counter() - t0)
        return t

    def _broadcast_stops(self, pri: PerRequestInfo, stops: set) -> None:
        peers = {w for ws_ in pri.worker_graph_to_workers.values() for w in ws_ if w != self.worker_id}
        for w in peers:
            self.comm.send(w, Message(WM.STOP_LOOPS, ipc.StopLoops(pri.request_id, set(stops), pri.partition_name)))

    def _walk_done(self, pri: PerRequestInfo) -> None:
        seq = {}
        for eng in self.engines.engines:
            if hasattr(eng, "get_per_label_seq_info"):
                seq.update(eng.get_per_label_seq_info(pri.request_id))
        # a rank reports the worker graphs whose first rank it is: the instance it follows is reported by its leader,
        # a single-rank group that shares this rank (a decoder beside a sharded model) by this rank itself
        led = [g for g in pri.worker_graph_ids
               if (pri.worker_graph_to_workers.get(g) or [self.worker_id])[0] == self.worker_id]
        if led or not self.is_tp_follower:
            body = ipc.WorkerGraphsDone(
                pri.request_id, led if self.is_tp_follower else list(pri.worker_graph_ids), True, dict(pri.persist),
                dict(pri.new_token_counts), seq,
                pri.partition_name, False, {}, pri.walk_state.loop_indices(),
                {"walk_s": time.perf_counter() - pri.t_start}, pri.fwd_info.graph_walk)
            if self._done_queue is not None:
                self._done_queue.append(body)       # sent once the batch that ended the walk is in the profile
            else:
                self._send_walk_done(body)
        pri.persist = {}
        pri.new_token_counts = {}
        for part, name in self._deferred_stream_end.pop((pri.request_id, pri.partition_name), []):
            dst = self.requests.get((pri.request_id, part))
            sb = dst.stream_buffers.get(name) if dst is not None else None
            if sb is not None:
                sb.signal_done()
                self._stream_dirty.add((pri.request_id, part))

    def _send_walk_done(self, body) -> None:
        if self.profile is not None:
            body.timings["profile"] = self.profile.pop(body.request_id)
        self.comm.send(self.conductor_id, Message(CM.WORKER_GRAPHS_DONE, body))

    # ------------------------------------------------------------------ failures
    def _fail_requests(self, errors: dict[str, str]) -> None:
        if not errors:
            return
        self.comm.send(self.conductor_id, Message(CM.FAIL_REQUESTS, ipc.FailRequests(dict(errors))))
        for rid in errors:
            for key in [k for k in self.requests if k[0] == rid]:
                pri = self.requests[key]
                if pri.in_flight:
                    pri.remove_pending = True
                else:
                    self._drop(key)

    def _handle_allocation_failure(self, batch: NodeBatch, out: NodeOutput) -> None:
        """Unwind the batch; free pages by offloading the request that holds the most, else back off."""
        eng = self.engines.engine_for(batch.node_name)
        rkeys = []
        for rid in batch.request_ids:
            pri = self.requests.get((rid, batch.partitions[rid]))
            if pri is None:
                continue
            pri.in_flight -= 1
            st = pri.walk_state.nodes[batch.node_name]
            st.running = False
            rkeys.append(_rk(pri))
        freed = 0
        if eng.can_offload():
            others = [k[0] for k in self.requests if k[0] not in batch.request_ids]
            victim = max(others or batch.request_ids, key=lambda r: eng.pages_of(r), default=None)
            if victim is not None:
                freed = eng.offload_request(victim)
        self.scheduler.hold(rkeys, 0.0 if freed else 0.05)
        for rk in rkeys:
            self.scheduler.mark_ready(batch.node_name, batch.graph_walk, rk)

    # ------------------------------------------------------------------ main loop
    def step(self, block_s: float = 0.0) -> bool:
        """One iteration of the main loop; returns True when something happened."""
        self.iterations += 1
        did = False
        T = self.phase_s
        t0 = time.perf_counter()
        msgs = self.comm.recv_or_wake(block_s) if block_s > 0 else self.comm.drain()
        t1 = time.perf_counter()
        T["wait"] += t1 - t0
        if msgs:
            self._process_messages(msgs)
            did = True
        t2 = time.perf_counter()
        T["messages"] += t2 - t1
        self._poll_stream_buffers()
        t3 = time.perf_counter()
        T["streams"] += t3 - t2
        if self._pipes:
            did |= self._advance_pipes()
            T["finish"] += time.perf_counter() - t3
        while True:
            # an engine with flights takes no other batch: its next one is either the speculative continuation or
            # whatever the scheduler picks once the queue has drained
            busy = {k for k in self.scheduler.ready if id(self.engines.engine_for(k[0])) in self._pipes} \
                if self._pipes else None
            nxt = self.scheduler.get_next_batch(exclude=busy)
            if nxt is None:
                break
            node, walk, rkeys = nxt
            tb = time.perf_counter()
            batch = self._build_node_batch(node, walk, rkeys)
            T["build"] += time.perf_counter() - tb
            if batch is None:
                continue
            if not self.is_tp_follower and (self.parallel_nodes is None or node in self.parallel_nodes):
                for f in self.tp_followers:
                    self.comm.send(f, Message(WM.SCHEDULE_TP, ipc.ScheduleTPNode(node, walk, list(rkeys))))
            did = True
            self._submit(batch)
            if self.gpu_thread is None:
                break
        if self.scheduler.stalled is not None:
            node, walk, rks = self.scheduler.stalled
            self.scheduler.stalled = None
            for rk in rks:
                rid, part = rk.split("|", 1)
                pri = self.requests.get((rid, part))
                st = pri.walk_state.nodes.get(node) if pri is not None else None
                log.warning("worker %s: %s of %s in walk %s: %s", self.worker_id, node, rid, walk,
                            "request not held" if pri is None else
                            f"walk here {pri.fwd_info.graph_walk}, node state "
                            f"{None if st is None else dict(done=st.done, running=st.running, missing=sorted(st.missing()))}")
        if not did and self._stall_log_s > 0 and time.monotonic() - self._last_stall_scan > self._stall_log_s:
            self._last_stall_scan = time.monotonic()
            self._log_stalled_requests()
        if self.heartbeat_s and time.monotonic() - self._last_beat > self.heartbeat_s:
            self._last_beat = time.monotonic()
            self.comm.send(self.conductor_id, Message(CM.HEARTBEAT, ipc.SetupDone(self.worker_id)))
        return did

    # ------------------------------------------------------------------ flights
    def _submit(self, batch: NodeBatch, speculative: bool = False, chain: int = 0) -> _Flight:
        eng = self.engines.engine_for(batch.node_name)
        self._next_fid += 1
        fl = _Flight(self._next_fid, batch, eng, speculative=speculative, chain=chain, t_submit=time.perf_counter())
        if self.trace is not None:
            self.trace.append((time.monotonic(), "submit", f"{batch.node_name}:{batch.graph_walk}", len(batch.request_ids),
                               int(speculative), fl.fid))
        if self.gpu_thread is None:          # synchronous mode: launch, wait, read back
            try:
                fl.pending = self._launch(fl)
            except Exception as e:  # noqa: BLE001
                fl.error = e
            self._finish(fl)
            return fl
        fl.fut = self.gpu_thread.submit(self._launch, fl)
        self._pipes.setdefault(id(eng), deque()).append(fl)
        return fl

    def _advance_pipes(self) -> bool:
        """Take finished launches, read back the batches whose results are there (in launch order per engine) and
        queue speculative continuations."""
        did = False
        for eid in list(self._pipes):
            pipe = self._pipes[eid]
            for fl in pipe:
                if fl.pending is None and fl.error is None and fl.fut.done():
                    try:
                        fl.pending = fl.fut.result()
                    except Exception as e:  # noqa: BLE001
                        fl.error = e
            # the continuation is queued FIRST (the sooner it sits behind the running batch, the less the GPU can
            # idle), then the batches whose results are there are read back
            if self._spec_enabled and 1 <= len(pipe) <= self._spec_depth:
                last = pipe[-1]
                if last.pending is not None and last.error is None and not last.spec_tried:
                    last.spec_tried = True
                    nb = self._build_speculative_batch(last, pipe)
                    if nb is not None:
                        self.spec_stats["launched"] += 1
                        self._submit(nb, speculative=True, chain=last.chain + 1)
                        did = True
            while pipe and (pipe[0].error is not None or (pipe[0].pending is not None and pipe[0].pending.ready())):
                self._finish(pipe.popleft())
                did = True
            if not pipe:
                del self._pipes[eid]
        return did

    def _build_speculative_batch(self, fl: _Flight, pipe) -> NodeBatch | None:
        """The next iteration of ``fl``'s loop node for the same requests, to be queued while ``fl`` still runs.
        None when the engine cannot continue from device-resident outputs, when some request may end its loop with
        the iteration in flight, when the chain is long enough, or when other work waits for this engine (a chain
        must not starve new requests: it is cut as soon as the scheduler holds anything else for the engine)."""
        b, pend, eng = fl.batch, fl.pending, fl.engine
        node, walk = b.node_name, b.graph_walk
        if any(f.batch.node_name != node or f.batch.graph_walk != walk or f.pending is None or f.error is not None
               or f.batch.request_ids != b.request_ids for f in pipe):
            return None
        queued_iters = sum(f.pending.iterations for f in pipe)      # iterations launched and not yet read back
        if fl.chain >= self._max_chain or pend.planned is None or pend.out.failed_requests or pend.out.allocation_failed:
            return None
        if not eng.can_speculate(node, walk):
            return None
        for k in self.scheduler.ready:
            if self.engines.engine_for(k[0]) is eng and self.scheduler._eligible(k):
                return None
        pris, remaining = [], []
        for rid in b.request_ids:
            pri = self.requests.get((rid, b.partitions[rid]))
            if pri is None or pri.remove_pending or pri.fwd_info.graph_walk != walk:
                return None
            if fl.speculative and fl.fid not in pri.spec.get(node, ()):
                return None              # this request left the loop: the chain ends here
            ws = pri.walk_state
            st = ws.nodes.get(node)
            if st is None or not st.running or not ws.can_speculate(node, ahead=len(pipe), chained=True):
                return None
            left = st.scope.loop.max_iters - st.scope.curr_iter - queued_iters
            if left < 1:
                return None
            pris.append(pri)
            remaining.append(left)
        infos = {}
        for pri, left in zip(pris, remaining):
            pri.fwd_info.step_metadata = dict(pri.fwd_info.step_metadata or {}, _loop_remaining=left)
            pri.walk_state.begin_speculation(node)
            pri.in_flight += 1
            pri.spec.setdefault(node, []).append(self._next_fid + 1)      # the id _submit gives the flight
            infos[pri.request_id] = pri.fwd_info
        nb = NodeBatch(node, walk, list(b.request_ids), {rid: {} for rid in b.request_ids}, infos, speculative=True)
        nb.partitions = dict(b.partitions)
        return nb

    def _cancel_speculation(self, fl: _Flight) -> None:
        """A speculative launch that queued nothing (page reservation failed): hand its requests back to the normal
        path."""
        self.spec_stats["cancelled"] += 1
        node = fl.batch.node_name
        for rid in fl.batch.request_ids:
            pri = self.requests.get((rid, fl.batch.partitions[rid]))
            if pri is None:
                continue
            pri.in_flight -= 1
            if fl.fid in pri.spec.get(node, ()):
                pri.spec[node].remove(fl.fid)
                pri.walk_state.rollback_speculation(node)
                if node in pri.spec_marked:          # iteration N was read back meanwhile: N+1 goes to the scheduler
                    pri.spec_marked.discard(node)
                    pri.walk_state.nodes[node].running = False
                    self._refresh_ready(pri)
            if pri.remove_pending and pri.in_flight == 0:
                self._drop((rid, pri.partition_name))

    def _finish(self, fl: _Flight) -> None:
        batch = fl.batch
        try:
            if fl.error is not None:
                raise fl.error
            out = fl.engine.collect_batch(fl.pending)
            dt = time.perf_counter() - fl.t_submit
            t_post = time.perf_counter()
            if self.trace is not None:
                self.trace.append((time.monotonic(), "collect", f"{batch.node_name}:{batch.graph_walk}",
                                   len(batch.request_ids), int(fl.speculative), fl.fid))
            out.timings["execute_s"] = dt
            rec = self.batches_by_node.setdefault(f"{batch.node_name}:{batch.graph_walk}", [0, 0, 0.0])
            rec[0] += 1
            rec[1] += len(batch.request_ids)
            rec[2] += dt
            self._done_queue = []
            self._emit_buf = []
            try:
                self._postprocess_batch(batch, out, fl)
            finally:
                done, self._done_queue = self._done_queue, None
                emits, self._emit_buf = self._emit_buf, None
                if len(emits) == 1:
                    self.comm.send(self.api_id, Message(ipc.ApiMessageType.RESULT_TENSORS, emits[0]))
                elif emits:
                    self.comm.send(self.api_id, Message(ipc.ApiMessageType.RESULT_TENSORS_BATCH,
                                                        ipc.ResultTensorsBatch(emits)))
            if self.profile is not None:
                tm = out.timings
                self.profile.record_batch(batch.node_name, batch.graph_walk, batch.request_ids,
                                          launch_s=tm.get("prepare_s", 0.0) + tm.get("plan_s", 0.0) + tm.get("forward_s", 0.0),
                                          flight_s=dt, post_s=tm.get("postprocess_s", 0.0) + time.perf_counter() - t_post,
                                          iterations=out.iterations, speculative=fl.speculative)
            for body in done:
                self._send_walk_done(body)
        except Exception as e:  # noqa: BLE001
            log.error("worker %s: batch %s failed: %s\n%s", self.worker_id, batch.node_name, e,
                      "".join(traceback.format_exception(type(e), e, e.__traceback__)))
            for rid in batch.request_ids:
                pri = self.requests.get((rid, batch.partitions[rid]))
                if pri is not None:
                    pri.in_flight = max(0, pri.in_flight - 1)
                    if fl.fid in pri.spec.get(batch.node_name, ()):
                        pri.spec[batch.node_name].remove(fl.fid)
            self._fail_requests({rid: f"{type(e).__name__}: {e}" for rid in batch.request_ids})

    def run(self) -> None:
        prof_dir = os.environ.get("MSTAR_PROFILE_WORKER")
        if prof_dir:          # host-side profile of the worker loop: one pstats file per worker
            import profile as _profile          # per-thread (sys.setprofile); cProfile's hooks are process-wide
            pr = _profile.Profile()
            try:
                pr.runcall(self._run_loop)
            finally:
                os.makedirs(prof_dir, exist_ok=True)
                pr.dump_stats(os.path.join(prof_dir, f"{self.worker_id}.pstats"))
            return
        self._run_loop()

    def _run_loop(self) -> None:
        # the launch thread and this loop share the interpreter lock: with the default 5 ms switch interval each
        # hand-over between them can stall a launch for milliseconds
        import sys
        sys.setswitchinterval(float(os.environ.get("MSTAR_PY_SWITCH_INTERVAL_SEC", "0.0002")))
        self.comm.send(self.conductor_id, Message(CM.SETUP_DONE, ipc.SetupDone(self.worker_id)))
        while self.running:
            if self._pipes:
                # batches are being launched or run on the GPU: sleep on the mailbox in short slices instead of
                # spinning on the GIL that the launch thread needs
                self.step(block_s=0.0003)
            else:
                self.step(block_s=0.0 if self.scheduler.has_ready() else 0.02)
        self.shutdown()

    def stats(self) -> dict:
        """Counters of this worker: host seconds by loop phase, batches per (node, walk), speculation, engine phases,
        bytes copied between host and device, CUDA-graph replays."""
        from ..utils import io_counters
        return {"worker": self.worker_id, "iterations": self.iterations,
                "phase_s": {k: round(v, 4) for k, v in self.phase_s.items()},
                "batches": {k: {"count": v[0], "requests": v[1], "seconds": round(v[2], 4)}
                            for k, v in self.batches_by_node.items()},
                "speculation": dict(self.spec_stats),
                "engines": [{"nodes": list(e.node_names), "phase_s": {k: round(v, 4) for k, v in e.phase_s.items()},
                             "graph_replays": getattr(e, "graph_hits", 0),
                             "decode_device_ms": round(getattr(e, "decode_device_ms", 0.0), 3),
                             "decode_steps": getattr(e, "decode_steps", 0)} for e in self.engines.engines],
                **({"trace": self.trace} if self.trace is not None else {}),
                **io_counters.snapshot()}

    def shutdown(self) -> None:
        if self.gpu_thread is not None:
            self.gpu_thread.shutdown(wait=True)
        stats_dir = os.environ.get("MSTAR_WORKER_STATS_DIR")
        if stats_dir:
            import json
            try:
                os.makedirs(stats_dir, exist_ok=True)
                with open(os.path.join(stats_dir, f"{self.worker_id}.json"), "w") as f:
                    json.dump(self.stats(), f)
            except Exception:  # noqa: BLE001
                log.exception("worker %s: could not write its stats", self.worker_id)
        if os.environ.get("MSTAR_WORKER_STATS"):
            log.warning("worker %s: loop iterations %d, host seconds by phase %s, batches (count, requests, seconds "
                        "from submission to read-back) %s, speculation %s, engine phases %s",
                        self.worker_id, self.iterations, {k: round(v, 3) for k, v in self.phase_s.items()},
                        {k: (v[0], v[1], round(v[2], 3)) for k, v in self.batches_by_node.items()}, self.spec_stats,
                        [{k: round(v, 3) for k, v in e.phase_s.items()} for e in self.engines.engines])


def _rk(pri: PerRequestInfo) -> str:
    return f"{pri.request_id}|{pri.partition_name}"


def _with_max_iters(loop, n: int):
    import copy
    c = copy.copy(loop)
    c.max_iters = n
    return c
