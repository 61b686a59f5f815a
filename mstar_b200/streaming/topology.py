"""Partitions: a model's walks may be grouped into asynchronously running partitions (LLM -> codec,
thinker -> talker -> vocoder) joined by streaming connections.

Reference counterparts: ``StreamingGraphEdge``, ``Connection``, ``PartitionTopology``
(mstar/streaming/topology.py:24-40), ``PartitionDefinition`` (mstar/conductor/request_info.py:92-103).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from ..graph.ir import GraphEdge
from .chunk_policy import ChunkPolicy


@dataclass
class StreamingGraphEdge(GraphEdge):
    target_partition: str = ""

    def __post_init__(self):
        self.is_streaming = True


@dataclass
class Connection:
    from_partition: str
    to_partition: str
    edge_name: str
    chunk_policy_factory: Callable[[], ChunkPolicy]


@dataclass
class PartitionTopology:
    partitions: list[str]
    connections: list[Connection] = field(default_factory=list)

    def incoming(self, partition: str) -> list[Connection]:
        return [c for c in self.connections if c.to_partition == partition]

    def outgoing(self, partition: str) -> list[Connection]:
        return [c for c in self.connections if c.from_partition == partition]


@dataclass
class PartitionDefinition:
    name: str
    graph_walks: list[str]
    initial_walk: str
    producer_partitions: list[str] = field(default_factory=list)
