"""Model-as-dataflow-graph IR. A model declares, per *walk* (prefill, decode, image_gen, ...), a ``GraphSection``
built from ``GraphNode`` leaves composed with ``Sequential``, ``Parallel`` and ``Loop``. Edges carry named
signals (tensor descriptors) between nodes; two special destinations send a signal to the client or nowhere.

The declarative classes here hold no per-request state: ``mstar_b200.graph.walk_state.WalkState`` instantiates
the run-time state of one request's walk from them.

Reference counterparts: ``TensorPointerInfo`` (mstar/graph/base.py:17-58), ``GraphEdge`` (:61-93), ``GraphNode``
(:222-358), ``Sequential`` (:361-412), ``Parallel`` (:415-453), ``Loop`` (:456-641), special destinations
(mstar/graph/special_destinations.py).
"""
from __future__ import annotations

import itertools as _itertools
import os as _os
import uuid as _uuid
from dataclasses import dataclass, field, replace

# Tensor ids must be unique across the processes of a deployment and are minted several times per request per decode
# step: a random per-process prefix plus a counter costs a fraction of uuid4 (which reads the kernel's random pool).
_UID_PREFIX = _os.urandom(6).hex()
_UID_COUNTER = _itertools.count()


def fast_uid() -> str:
    return f"{_UID_PREFIX}{next(_UID_COUNTER):x}"


EMIT_TO_CLIENT = "__emit_to_client__"
EMPTY_DESTINATION = "__empty_destination__"
SPECIAL_DESTINATIONS = (EMIT_TO_CLIENT, EMPTY_DESTINATION)


@dataclass
class TensorPointerInfo:
    """Descriptor of a tensor held by some entity's tensor store (worker or API server)."""
    dims: list[int]
    dtype: str
    nbytes: int
    address: int = 0
    stride: list[int] = field(default_factory=list)
    uuid: str = field(default_factory=fast_uid)
    source_session_id: str = ""
    source_entity: str = ""
    offset: int = 0
    source_tp_size: int = 1
    source_tp_rank: int = 0
    shm_segment: str | None = None
    shm_offset: int = 0
    device_index: int = -1          # >= 0: lives on that GPU (peer-copyable over NVLink)
    cuda_ipc: tuple | None = None   # CUDA IPC handle of the producer's allocation for cross-process GPU reads

    def clone(self) -> "TensorPointerInfo":
        return replace(self, dims=list(self.dims), stride=list(self.stride))

    def __reduce__(self):      # compact pickling: these cross process boundaries many times per decode step
        return (_tpi_from_tuple, ((self.dims, self.dtype, self.nbytes, self.address, self.stride, self.uuid,
                                   self.source_session_id, self.source_entity, self.offset, self.source_tp_size,
                                   self.source_tp_rank, self.shm_segment, self.shm_offset, self.device_index,
                                   self.cuda_ipc),))


def _tpi_from_tuple(t):
    return TensorPointerInfo(*t)


@dataclass
class GraphEdge:
    next_node: str
    name: str
    tensor_info: list[TensorPointerInfo] = field(default_factory=list)
    persist: bool = False               # kept by the conductor across walks of the request
    conductor_new_token: bool = False   # counts toward the request's output-token budget
    is_streaming: bool = False          # accumulates in the consumer's stream buffer
    output_modality: str = ""           # for EMIT_TO_CLIENT edges: text | image | video | audio
    final_stream_chunk: bool = False    # set on the synthetic edge that carries a stream's last chunk
    total_fanin: int = 1                # sharded producers: how many shards make the signal complete
    shard_dim: int | None = None

    def key(self) -> tuple[str, str]:
        return (self.name, self.next_node)

    def clone(self, with_tensors: bool = True) -> "GraphEdge":
        return GraphEdge(self.next_node, self.name, list(self.tensor_info) if with_tensors else [], self.persist,
                         self.conductor_new_token, self.is_streaming, self.output_modality, self.final_stream_chunk,
                         self.total_fanin, self.shard_dim)


@dataclass
class IOSignature:
    ext_inputs: set[tuple[str, str]]          # (signal name, consumer node)
    ext_outputs: list[GraphEdge]
    loop_back: set[tuple[str, str]]           # signals that feed an earlier (or the same) node


class GraphSection:
    def nodes(self) -> dict[str, "GraphNode"]:
        raise NotImplementedError

    def loops(self) -> dict[str, "Loop"]:
        raise NotImplementedError

    def signature(self) -> IOSignature:
        raise NotImplementedError

    def children(self) -> list["GraphSection"]:
        return []

    # reference-compatible spellings
    def get_nodes(self):
        return self.nodes()

    def get_loops(self):
        return self.loops()

    def get_inputs_outputs(self):
        return self.signature()


@dataclass
class GraphNode(GraphSection):
    name: str
    input_names: set[str]
    outputs: list[GraphEdge] = field(default_factory=list)
    consumes_stream: bool = False
    enable_async_scheduling: bool = True     # may the worker speculate iteration N+1 while N runs?
    streaming_inputs: set[str] = field(default_factory=set)

    def __post_init__(self):
        self.input_names = set(self.input_names)
        self.streaming_inputs = set(self.streaming_inputs)
        if self.streaming_inputs:
            self.consumes_stream = True

    def nodes(self):
        return {self.name: self}

    def loops(self):
        return {}

    def signature(self) -> IOSignature:
        back = {(e.name, self.name) for e in self.outputs if e.next_node == self.name}
        return IOSignature(ext_inputs={(n, self.name) for n in self.input_names if (n, self.name) not in back},
                           ext_outputs=[e for e in self.outputs if e.next_node != self.name], loop_back=back)


class _Composite(GraphSection):
    sections: list[GraphSection]

    def nodes(self):
        out: dict[str, GraphNode] = {}
        for s in self.sections:
            for k, v in s.nodes().items():
                if k in out:
                    raise ValueError(f"duplicate node name {k!r} in one walk")
                out[k] = v
        return out

    def loops(self):
        out: dict[str, Loop] = {}
        for s in self.sections:
            out.update(s.loops())
        return out

    def children(self):
        return list(self.sections)


@dataclass
class Sequential(_Composite):
    sections: list[GraphSection]

    def signature(self) -> IOSignature:
        seen_nodes: set[str] = set()
        ext_in: set[tuple[str, str]] = set()
        back: set[tuple[str, str]] = set()
        outs: list[GraphEdge] = []
        for sec in self.sections:
            sig = sec.signature()
            back |= sig.loop_back
            # outputs of this section that point at an earlier section are loop-backs
            back |= {e.key() for e in sig.ext_outputs if e.next_node in seen_nodes}
            ext_in |= sig.ext_inputs
            outs.extend(sig.ext_outputs)
            internal = {e.key() for e in outs if e.key() in ext_in}
            outs = [e for e in outs if e.key() not in internal and e.key() not in back]
            ext_in -= internal | back
            seen_nodes |= set(sec.nodes())
        return IOSignature(ext_in, outs, back)


@dataclass
class Parallel(_Composite):
    sections: list[GraphSection]

    def signature(self) -> IOSignature:
        sigs = [s.signature() for s in self.sections]
        produced = {e.key() for s in sigs for e in s.ext_outputs}
        consumed = {k for s in sigs for k in s.ext_inputs}
        internal = produced & consumed
        back: set[tuple[str, str]] = set()
        ext_in: set[tuple[str, str]] = set()
        outs: list[GraphEdge] = []
        for s in sigs:
            back |= s.loop_back
            ext_in |= s.ext_inputs - internal
            outs.extend(e for e in s.ext_outputs if e.key() not in internal)
        return IOSignature(ext_in, outs, back)


@dataclass
class Loop(GraphSection):
    """Repeat ``section`` until ``max_iters`` iterations ran or the loop is told to stop. ``outputs`` leave the
    loop with the tensors of the LAST iteration; ``accumulated_outputs`` with the tensors of EVERY iteration.
    Inputs that come from outside the loop are kept and re-delivered at the start of every iteration."""
    section: GraphSection
    max_iters: int
    outputs: list[GraphEdge] = field(default_factory=list)
    name: str = field(default_factory=lambda: "loop_" + _uuid.uuid4().hex[:8])
    accumulated_outputs: list[GraphEdge] = field(default_factory=list)

    def __post_init__(self):
        sig = self.section.signature()
        self.external_inputs = set(sig.ext_inputs)
        self.loop_back_inputs = set(sig.loop_back)
        producible = {e.name for e in sig.ext_outputs} | {n for n, _ in sig.loop_back}
        self.outputs = [e for e in self.outputs if e.name in producible]
        self.accumulated_outputs = [e for e in self.accumulated_outputs if e.name in producible]
        both = {e.name for e in self.outputs} & {e.name for e in self.accumulated_outputs}
        if both:
            raise ValueError(f"Loop outputs and accumulated_outputs overlap: {sorted(both)}")

    def nodes(self):
        return self.section.nodes()

    def loops(self):
        d = dict(self.section.loops())
        d[self.name] = self
        return d

    def children(self):
        return [self.section]

    def signature(self) -> IOSignature:
        sig = self.section.signature()
        return IOSignature(set(sig.ext_inputs), list(self.outputs) + list(self.accumulated_outputs),
                           set(sig.loop_back))


def entities_of(section: GraphSection) -> list[GraphSection]:
    """The nodes and loops that a section manages directly (loops hide what is inside them)."""
    if isinstance(section, (GraphNode, Loop)):
        return [section]
    out: list[GraphSection] = []
    for c in section.children():
        out.extend(entities_of(c))
    return out


def restrict_section(section: GraphSection, keep: set[str]) -> GraphSection | None:
    """The part of a walk that one worker runs: same composition, only the nodes in ``keep`` (None when the
    section has none of them). Loops keep their name and iteration budget, so that workers sharing a loop count
    iterations alike; edges that leave the kept set are routed to their owners by the worker."""
    if isinstance(section, GraphNode):
        return section if section.name in keep else None
    if isinstance(section, Loop):
        inner = restrict_section(section.section, keep)
        if inner is None:
            return None
        part = Loop(inner, section.max_iters, [e.clone() for e in section.outputs], section.name,
                    [e.clone() for e in section.accumulated_outputs])
        # what is a loop-back and what comes from outside is a property of the WHOLE loop: a signal fed back by a
        # node on another worker must not look like an outside input here (it would be re-delivered every iteration)
        part.loop_back_inputs = {k for k in section.loop_back_inputs if k[1] in keep}
        part.external_inputs = {k for k in section.external_inputs if k[1] in keep}
        return part
    kids = [k for k in (restrict_section(c, keep) for c in section.children()) if k is not None]
    if not kids:
        return None
    if len(kids) == 1:
        return kids[0]
    return type(section)(kids)
