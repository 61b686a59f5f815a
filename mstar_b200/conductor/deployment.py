"""Wiring of a deployment: parse the YAML config, build the model, start the conductor and one worker per rank.

Two modes:
  * ``in_process=True``  — conductor and workers as threads of this process over in-process mailboxes (CPU tests,
    single-GPU serving without process hops);
  * ``in_process=False`` — one OS process per worker (``cuda:{rank}``) and one for the conductor, talking over the
    C++ shared-memory mesh; TP / SP ranks join NCCL process groups and the symmetric heap.

Reference counterparts: worker spawn / shutdown in the conductor (mstar/conductor/conductor.py:82-152,419-473), the
conductor process target (mstar/api_server/entrypoint.py:55-113), YAML keys (docs/serving.rst:164-181).
"""
from __future__ import annotations

import logging
import multiprocessing as mp
import os
import signal
import threading
import uuid

import torch
import yaml

from ..communication.communicator import LocalCommunicator, make_communicator
from ..communication.tensors import TensorCommunicationManager
from ..models.registry import get_model_class
from ..worker.engine_manager import EngineManager
from ..worker.worker import Worker
from .conductor import Conductor, worker_id_of

log = logging.getLogger("mstar.deploy")


def load_config(path_or_dict) -> dict:
    if isinstance(path_or_dict, dict):
        cfg = dict(path_or_dict)
    else:
        with open(path_or_dict) as f:
            cfg = yaml.safe_load(f)
    cfg.setdefault("node_groups", [])
    cfg.setdefault("model_kwargs", {})
    return cfg


def build_model(cfg: dict):
    cls = get_model_class(cfg["model"])
    return cls(model_dir=cfg.get("model_dir"), skip_weight_loading=cfg.get("skip_weight_loading", cfg.get("model_dir") is None),
               **cfg.get("model_kwargs", {}))


def _device_for(rank: int):
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


def build_worker(cfg: dict, model, rank: int, comm, *, prefix: str, async_gpu: bool = True, dist_init: str | None = None,
                 heartbeat_s: float = 0.0) -> Worker:
    from ..parallel.comm import CommGroup, WorkerParallelGroups
    wgs = model.get_worker_graphs(cfg["node_groups"])
    mine = [wg for wg in wgs if rank in wg.ranks]
    node_names = sorted({n for wg in mine for n in wg.node_names})
    device = _device_for(rank)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    world = 1 + max(r for wg in wgs for r in wg.ranks)
    tp_group = sp_group = None
    par = [wg for wg in mine if wg.tp_size * wg.sp_size > 1]
    if par and dist_init:
        # the process group spans only the ranks that belong to some tensor- / sequence-parallel instance, numbered in
        # rank order: a rank that runs single-GPU nodes only (an encoder, a codec) never joins, so it cannot hold
        # the others' rendezvous up
        dist_ranks = sorted({r for w in wgs if w.tp_size * w.sp_size > 1 for r in w.ranks})
        dr = {r: i for i, r in enumerate(dist_ranks)}
        groups = WorkerParallelGroups(dr[rank], len(dist_ranks))
        _group_for = groups.group_for
        groups.group_for = lambda ranks: _group_for(tuple(dr[r] for r in ranks))
        def instance_tp_major(w):
            # all ranks of the instance, tensor-parallel index slowest: shard i of a weight cut tp*sp ways is the
            # sp-th part of tensor-parallel shard t (the head order that Ulysses produces inside a TP shard)
            return tuple(w.ranks[s * w.tp_size + t] for t in range(w.tp_size) for s in range(w.sp_size))
        pw = [w for w in wgs if w.tp_size * w.sp_size > 1]
        tuples = sorted({tuple(dr[x] for x in wg.tp_ranks(r)) for wg in pw for r in wg.ranks} |
                        {tuple(dr[x] for x in wg.sp_ranks(r)) for wg in pw for r in wg.ranks} |
                        {tuple(dr[x] for x in instance_tp_major(wg)) for wg in pw if wg.tp_size > 1 and wg.sp_size > 1})
        groups.init_dist(dist_init, all_rank_tuples=[t for t in tuples if len(t) > 1])
        wg = par[0]
        tp_group = groups.group_for(wg.tp_ranks(rank))
        sp_group = groups.group_for(wg.sp_ranks(rank))
        inst = (groups.group_for(instance_tp_major(wg)) if wg.tp_size > 1 and wg.sp_size > 1
                else (tp_group if wg.sp_size == 1 else sp_group))
        tp_group.instance = sp_group.instance = inst
        if device.type == "cuda":
            from ..parallel.symm import attach_symmetric_heap
            # the sequence-parallel group's heap holds the Ulysses exchange buffers (q / k / v of this rank's heads
            # over the full sequence and the attention output of its rows): hundreds of MB at video sizes
            user_mb = int(os.environ.get("MSTAR_SYMM_USER_MB", "1024" if wg.sp_size > 1 else "64"))
            for g in {id(x): x for x in (tp_group, sp_group, inst)}.values():
                if g.size > 1 and g.symm is None:
                    attach_symmetric_heap(g, device, user_bytes=(user_mb if g is sp_group else 64) << 20)
    tensors = TensorCommunicationManager(worker_id_of(rank), device, arena_prefix=prefix)
    kv = cfg.get("kv_cache", {}) or {}
    em = EngineManager(model, device, node_names, tp_group=tp_group, sp_group=sp_group, kv_overrides=kv,
                       max_batch=int(cfg.get("max_batch_size", 64)), use_cuda_graphs=cfg.get("use_cuda_graphs"))
    from ..worker.engine_manager import register_kv_engines
    register_kv_engines(worker_id_of(rank), em)
    n2w: dict[str, list[str]] = {}
    for wg in wgs:
        for n in wg.node_names:
            for r in wg.ranks:
                n2w.setdefault(n, [])
                if worker_id_of(r) not in n2w[n]:
                    n2w[n].append(worker_id_of(r))
    # the ranks of one model instance (tp x sp) run every batch in lockstep behind the instance's first rank
    leader_of = {r: wg.ranks[0] for wg in mine for r in wg.ranks if wg.tp_size * wg.sp_size > 1}
    followers = [worker_id_of(r) for wg in mine if wg.tp_size * wg.sp_size > 1 and wg.ranks[0] == rank
                 for r in wg.ranks[1:]]
    is_follower = rank in leader_of and leader_of[rank] != rank
    # a node that appears in several node groups with different walk filters is split by walk (prefill / decode
    # disaggregation): only then do persisted tensors have to be readable from other processes
    walks_of: dict[str, set] = {}
    for g in cfg["node_groups"]:
        for n in g.get("node_names", []):
            walks_of.setdefault(n, set()).add(tuple(sorted(g.get("graph_walks") or [])))
    split_by_walk = any(len(v) > 1 for v in walks_of.values())
    # the walks in which THIS rank runs each of its nodes (None: every walk)
    node_walks: dict[str, set | None] = {}
    for wg in mine:
        for n in wg.node_names:
            if wg.graph_walks is None or node_walks.get(n, set()) is None:
                node_walks[n] = None
            else:
                node_walks.setdefault(n, set()).update(wg.graph_walks)
    return Worker(worker_id_of(rank), rank, model, node_names, comm, tensors, em, node_to_workers=n2w,
                  # persisted tensors come back from the conductor in a later walk: to another worker when a node is
                  # split by walk, and to the other ranks of a tensor- / sequence-parallel instance always
                  publish_persisted=split_by_walk or bool(followers), node_walks=node_walks,
                  parallel_nodes={n for wg in par for n in wg.node_names},
                  instance_workers={worker_id_of(r) for wg in par for r in wg.ranks},
                  tp_followers=followers, is_tp_follower=is_follower, max_batch_size=int(cfg.get("max_batch_size", 64)),
                  async_gpu=async_gpu, heartbeat_s=heartbeat_s, log_stats=bool(cfg.get("log_stats")))


def _worker_process_target(cfg, rank, prefix, dist_init, heartbeat_s):
    import faulthandler
    faulthandler.enable()
    if os.environ.get("MSTAR_DUMP_STACKS_S"):        # debugging aid: every thread's stack of this worker after N seconds
        faulthandler.dump_traceback_later(float(os.environ["MSTAR_DUMP_STACKS_S"]), repeat=False)
    signal.signal(signal.SIGTERM, lambda *_: (_ for _ in ()).throw(SystemExit(0)))
    logging.basicConfig(level=os.environ.get("MSTAR_LOG_LEVEL", "INFO"))
    # a launcher may have pinned OMP_NUM_THREADS to 1 for its own ranks; weight initialisation / loading and host-side
    # tensor work in a worker want a few cores
    try:
        n_workers = len({r for g in cfg.get("node_groups", []) for r in g.get("ranks", [0])}) or 1
        torch.set_num_threads(max(1, min(16, (os.cpu_count() or 8) // n_workers)))
    except Exception:  # noqa: BLE001
        pass
    if os.environ.get("MSTAR_CUDNN_BENCHMARK", "0") == "1":
        # library convolutions (codecs, VAEs): let cuDNN time its algorithms on the first call of each shape, which
        # happens in the eager warm-up run before a shape's graph is captured
        torch.backends.cudnn.benchmark = True
    model = build_model(cfg)
    comm = make_communicator(worker_id_of(rank), "shm", prefix)
    w = build_worker(cfg, model, rank, comm, prefix=prefix, dist_init=dist_init, heartbeat_s=heartbeat_s)
    try:
        w.run()
    finally:
        comm.close()


def _conductor_process_target(cfg, prefix, heartbeat_timeout_s):
    import faulthandler
    faulthandler.enable()
    if os.environ.get("MSTAR_DUMP_STACKS_S"):
        faulthandler.dump_traceback_later(float(os.environ["MSTAR_DUMP_STACKS_S"]), repeat=False)
    signal.signal(signal.SIGTERM, lambda *_: (_ for _ in ()).throw(SystemExit(0)))
    logging.basicConfig(level=os.environ.get("MSTAR_LOG_LEVEL", "INFO"))
    model = build_model(cfg)
    comm = make_communicator("conductor", "shm", prefix)
    c = Conductor(cfg, model, comm, heartbeat_timeout_s=heartbeat_timeout_s)
    try:
        c.run()
    finally:
        comm.close()


class Deployment:
    def __init__(self, config, *, in_process: bool = True, async_gpu: bool = True, heartbeat_s: float = 0.0,
                 heartbeat_timeout_s: float = 0.0):
        self.cfg = load_config(config)
        self.in_process = in_process
        self.prefix = "mstar_" + uuid.uuid4().hex[:10]
        self.model = build_model(self.cfg)
        self.threads: list[threading.Thread] = []
        self.procs: list[mp.Process] = []
        self.workers: list[Worker] = []
        self.conductor: Conductor | None = None
        ranks = sorted({r for g in self.cfg["node_groups"] for r in g.get("ranks", [0])})
        if in_process:
            self.hub = LocalCommunicator.new_hub()
            self.api_comm = LocalCommunicator("api", self.hub)
            self.conductor = Conductor(self.cfg, self.model, LocalCommunicator("conductor", self.hub),
                                       heartbeat_timeout_s=heartbeat_timeout_s)
            for r in ranks:
                w = build_worker(self.cfg, self.model, r, LocalCommunicator(worker_id_of(r), self.hub),
                                 prefix=self.prefix, async_gpu=async_gpu, heartbeat_s=heartbeat_s)
                self.workers.append(w)
            self.threads = [threading.Thread(target=self.conductor.run, daemon=True, name="conductor")]
            self.threads += [threading.Thread(target=w.run, daemon=True, name=w.worker_id) for w in self.workers]
        else:
            ctx = mp.get_context("spawn")
            self.api_comm = make_communicator("api", "shm", self.prefix)
            needs_dist = any(int(g.get("tp_size", 1)) * int(g.get("sp_size", 1)) > 1 for g in self.cfg["node_groups"])
            dist_init = None
            if needs_dist:
                import socket
                s = socket.socket()
                s.bind(("127.0.0.1", 0))
                dist_init = f"tcp://127.0.0.1:{s.getsockname()[1]}"
                s.close()
            self.procs.append(ctx.Process(target=_conductor_process_target, args=(self.cfg, self.prefix, heartbeat_timeout_s),
                                          daemon=True))
            for r in ranks:
                self.procs.append(ctx.Process(target=_worker_process_target,
                                              args=(self.cfg, r, self.prefix, dist_init, heartbeat_s), daemon=True))

    def start(self) -> None:
        for t in self.threads:
            t.start()
        for p in self.procs:
            p.start()

    def shutdown(self, timeout_s: float = 10.0) -> None:
        from ..utils.ipc_format import ConductorMessageType, Message
        try:
            self.api_comm.send("conductor", Message(ConductorMessageType.SHUTDOWN, None))
        except Exception:  # noqa: BLE001
            pass
        for t in self.threads:
            t.join(timeout_s)
        for p in self.procs:
            p.join(timeout_s)
            if p.is_alive():
                p.terminate()
                p.join(2.0)
                if p.is_alive():
                    p.kill()
        if not self.in_process:
            self.api_comm.close()
            from ..communication.arena import sweep_orphans
            sweep_orphans(self.prefix)
