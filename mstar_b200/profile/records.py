"""Per-request profile: what one request cost, stage by stage. Workers accumulate node timings and tensor transfers
per request (``WorkerProfile``), hand them to the conductor with every finished walk, the conductor adds its own
checkpoints, and the API server merges everything with the client-facing timestamps and prints the tree when the
server runs with ``--log-stats`` (or writes it to ``--log-stats-file``).

A node execution is split the way the pipelined worker runs it:
  * ``launch_s``   host time to prepare inputs, plan and queue the batch's GPU work (the launch thread);
  * ``flight_s``   from submission to the moment the results were on the host (GPU time plus queueing behind
                   batches launched ahead of it: with speculative launches several flights overlap, so flights of
                   one request are not additive);
  * ``post_s``     host time of per-request postprocessing and routing, shared equally by the batch's requests.

Reference counterparts: ``RequestProfile`` and its parts (mstar/profile/format.py:6-89), ``WorkerProfileInfo``
(mstar/profile/worker.py:12-106).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field


@dataclass
class NodeTiming:
    node: str
    walk: str
    worker: str = ""
    executions: int = 0
    iterations: int = 0           # loop iterations covered (a decode burst covers several per execution)
    speculative: int = 0          # executions that were queued before their predecessor had been read back
    batch_rows: int = 0           # sum of batch sizes the request ran in (executions x mean batch)
    launch_s: float = 0.0
    flight_s: float = 0.0
    post_s: float = 0.0

    def add(self, o: "NodeTiming") -> None:
        self.executions += o.executions
        self.iterations += o.iterations
        self.speculative += o.speculative
        self.batch_rows += o.batch_rows
        self.launch_s += o.launch_s
        self.flight_s += o.flight_s
        self.post_s += o.post_s


@dataclass
class Transfer:
    direction: str                # "tx" (published for another entity) | "rx" (fetched from another entity)
    edge: str
    src: str
    dst: str
    count: int = 0
    nbytes: int = 0
    seconds: float = 0.0


@dataclass
class RequestProfile:
    request_id: str
    checkpoints: dict = field(default_factory=dict)       # name -> seconds since the request was received
    inputs: dict = field(default_factory=dict)            # modality -> [count, bytes]
    outputs: dict = field(default_factory=dict)           # modality -> [count, bytes]
    nodes: list = field(default_factory=list)             # NodeTiming
    transfers: list = field(default_factory=list)         # Transfer
    tokens_out: int = 0

    def merge_worker(self, d: dict) -> None:
        """Fold in one ``WorkerProfile.pop`` result (plain dicts, as they travel on the mesh)."""
        for n in d.get("nodes", []):
            nt = NodeTiming(**n)
            cur = next((x for x in self.nodes if (x.node, x.walk, x.worker) == (nt.node, nt.walk, nt.worker)), None)
            if cur is None:
                self.nodes.append(nt)
            else:
                cur.add(nt)
        for t in d.get("transfers", []):
            tr = Transfer(**t)
            cur = next((x for x in self.transfers if (x.direction, x.edge, x.src, x.dst) ==
                        (tr.direction, tr.edge, tr.src, tr.dst)), None)
            if cur is None:
                self.transfers.append(tr)
            else:
                cur.count += tr.count
                cur.nbytes += tr.nbytes
                cur.seconds += tr.seconds

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "RequestProfile":
        p = cls(d.get("request_id", ""), dict(d.get("checkpoints", {})), dict(d.get("inputs", {})),
                dict(d.get("outputs", {})), tokens_out=int(d.get("tokens_out", 0)))
        p.nodes = [NodeTiming(**n) for n in d.get("nodes", [])]
        p.transfers = [Transfer(**t) for t in d.get("transfers", [])]
        return p


class WorkerProfile:
    """Worker-side accumulation, keyed by request. ``pop`` empties a request's record (sent with a finished walk)."""

    def __init__(self, worker_id: str):
        self.worker_id = worker_id
        self._nodes: dict[str, dict[tuple[str, str], NodeTiming]] = {}
        self._xfer: dict[str, dict[tuple, Transfer]] = {}

    def record_batch(self, node: str, walk: str, request_ids: list[str], *, launch_s: float, flight_s: float,
                     post_s: float, iterations: dict | None = None, speculative: bool = False) -> None:
        n = max(1, len(request_ids))
        for rid in request_ids:
            per = self._nodes.setdefault(rid, {})
            nt = per.get((node, walk))
            if nt is None:
                nt = per[(node, walk)] = NodeTiming(node, walk, self.worker_id)
            nt.executions += 1
            nt.iterations += int((iterations or {}).get(rid, 1))
            nt.speculative += int(speculative)
            nt.batch_rows += n
            nt.launch_s += launch_s
            nt.flight_s += flight_s
            nt.post_s += post_s / n

    def record_transfer(self, request_id: str, direction: str, edge: str, src: str, dst: str, nbytes: int,
                        seconds: float) -> None:
        per = self._xfer.setdefault(request_id, {})
        key = (direction, edge, src, dst)
        t = per.get(key)
        if t is None:
            t = per[key] = Transfer(direction, edge, src, dst)
        t.count += 1
        t.nbytes += int(nbytes)
        t.seconds += seconds

    def pop(self, request_id: str) -> dict:
        nodes = self._nodes.pop(request_id, {})
        xfer = self._xfer.pop(request_id, {})
        return {"nodes": [asdict(v) for v in nodes.values()], "transfers": [asdict(v) for v in xfer.values()]}

    def drop(self, request_id: str) -> None:
        self._nodes.pop(request_id, None)
        self._xfer.pop(request_id, None)
