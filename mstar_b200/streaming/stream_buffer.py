"""Consumer-side buffer of a streaming edge: items arrive one by one (possibly out of order with respect to
their announcements), a ``ChunkPolicy`` gates when the consuming node may run, and the last chunk is flagged so
that the stream closes exactly once.

Reference counterparts: ``StreamChunk`` / ``StreamBuffer`` (mstar/streaming/stream_buffer.py), final-flush
behaviour pinned by test/modular/test_stream_buffer_final_flush.py.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

from .chunk_policy import ChunkPolicy


@dataclass
class StreamChunk:
    data: dict
    chunk_index: int
    start_offset: int = 0        # global index of the chunk's first item
    is_final: bool = False


@dataclass
class StreamBuffer:
    request_id: str
    edge_name: str
    from_partition: str
    policy: ChunkPolicy
    producer_done: bool = False
    _announced: deque = field(default_factory=deque)    # tensor ids in arrival-announcement order
    _arrived: dict = field(default_factory=dict)        # tensor id -> item, waiting for its turn
    _items: list = field(default_factory=list)          # in-order items not yet dropped
    _consumed: int = 0
    _chunks: int = 0
    _n_announced: int = 0
    _n_buffered: int = 0
    _final_emitted: bool = False
    _parked_edges: deque = field(default_factory=deque)

    # ---- producer side ----
    def pre_read_register(self, tensor_id: str) -> None:
        """An item was announced (its descriptor arrived); its payload may land later."""
        self._announced.append(tensor_id)
        self._n_announced += 1

    def put(self, tensor_id: str, item) -> None:
        if tensor_id not in self._announced and tensor_id not in self._arrived:
            self.pre_read_register(tensor_id)
        self._arrived[tensor_id] = item

    def signal_done(self) -> None:
        self.producer_done = True

    # ---- parked graph edges (chunks handed back after a rolled-back readiness check) ----
    def store_uningested_edge(self, edge) -> None:
        self._parked_edges.append(edge)

    def pop_waiting_edge(self):
        return self._parked_edges.popleft() if self._parked_edges else None

    # ---- consumer side ----
    def _drain_in_order(self) -> None:
        while self._announced and self._announced[0] in self._arrived:
            self._items.append(self._arrived.pop(self._announced.popleft()))
            self._n_buffered += 1

    def _all_arrived(self) -> bool:
        return self.producer_done and self._n_buffered >= self._n_announced

    def __len__(self) -> int:
        self._drain_in_order()
        return len(self._items)

    def has_chunk_ready(self) -> bool:
        self._drain_in_order()
        n = len(self._items)
        if not self._all_arrived():
            return self.policy.is_ready(n)
        # producer finished: flush what is left; if nothing is left, still emit ONE final (empty) chunk
        return n > 0 or self.policy.continue_after_producer_done() or not self._final_emitted

    def pop_chunk(self) -> StreamChunk:
        self._drain_in_order()
        n = len(self._items)
        offset = self._consumed
        if self._all_arrived() and not self.policy.is_ready(n):
            items, adv = list(self._items), n
            self._items = []
        else:
            adv = self.policy.next_chunk_size(n)
            items = self._items[:self.policy.window_size()]
            self._items = self._items[adv:]
        self._consumed += adv
        self.policy.register_chunk(adv)
        final = self._all_arrived() and not self._items and not self.policy.continue_after_producer_done()
        if final:
            self._final_emitted = True
        chunk = StreamChunk(self._collate(items), self._chunks, offset, final)
        self._chunks += 1
        return chunk

    @staticmethod
    def _collate(items: list) -> dict:
        if not items:
            return {"data": None}
        if all(isinstance(i, torch.Tensor) for i in items):
            return {"data": items[0] if len(items) == 1 else torch.stack(items)}
        if any(isinstance(i, torch.Tensor) for i in items):      # single-token tensors mixed with burst ints
            return {"data": [int(i.reshape(-1)[0]) if isinstance(i, torch.Tensor) else i for i in items]}
        return {"data": items}
