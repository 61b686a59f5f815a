"""Signals between node groups of different tensor-parallel size: when a producer group of size Tp feeds a
consumer group of size Tc, a *replicated* signal is read from one producer rank per consumer rank, a *sharded*
signal (split along ``shard_dim``) is re-cut by byte ranges on the leading shard dimension.

Reference counterpart: ``ShardingConfig.compute_fanout`` / ``fanout_graph_edges`` / ``compute_fanin``
(mstar/distributed/base.py:55-342), pinned by test/distributed/test_sharding_config.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..graph.ir import GraphEdge, TensorPointerInfo


@dataclass
class ShardingConfig:
    sharded_signals: dict[str, int] = field(default_factory=dict)     # signal name -> shard dim (only dim 0 supported)

    def is_sharded(self, name: str) -> bool:
        return name in self.sharded_signals

    def compute_fanout(self, name: str, src_tp: int, dst_tp: int) -> list[list[tuple[int, float, float]]]:
        """For every destination rank: list of (source rank, start fraction, end fraction) of the source shard to
        read. Replicated signals: one whole read from source rank ``d % src_tp``."""
        plan = []
        for d in range(dst_tp):
            if not self.is_sharded(name):
                plan.append([(d % src_tp, 0.0, 1.0)])
                continue
            lo, hi = d / dst_tp, (d + 1) / dst_tp          # destination's slice of the whole tensor
            reads = []
            for s in range(src_tp):
                slo, shi = s / src_tp, (s + 1) / src_tp
                a, b = max(lo, slo), min(hi, shi)
                if b > a + 1e-12:
                    reads.append((s, (a - slo) * src_tp, (b - slo) * src_tp))
            plan.append(reads)
        return plan

    def compute_fanin(self, name: str, src_tp: int, dst_tp: int) -> int:
        """How many partial descriptors a destination rank must collect before the signal is complete."""
        return max(len(r) for r in self.compute_fanout(name, src_tp, dst_tp))

    def fanout_graph_edges(self, edge: GraphEdge, shards: list[list[TensorPointerInfo]], dst_tp: int) -> list[GraphEdge]:
        """``shards[s]`` = descriptors produced by source rank s. Returns one edge per destination rank whose
        descriptors carry byte offsets / sizes of the part to read."""
        src_tp = len(shards)
        plan = self.compute_fanout(edge.name, src_tp, dst_tp)
        out = []
        for d, reads in enumerate(plan):
            e = edge.clone(with_tensors=False)
            e.total_fanin = len(reads)
            e.shard_dim = self.sharded_signals.get(edge.name)
            for s, a, b in reads:
                for ti in shards[s]:
                    c = ti.clone()
                    rows = ti.dims[0] if ti.dims else 1
                    r0, r1 = int(round(a * rows)), int(round(b * rows))
                    row_bytes = ti.nbytes // max(1, rows)
                    c.offset = r0 * row_bytes
                    c.nbytes = (r1 - r0) * row_bytes
                    if c.dims:
                        c.dims = [r1 - r0] + list(ti.dims[1:])
                    c.source_tp_size, c.source_tp_rank = src_tp, s
                    e.tensor_info.append(c)
            out.append(e)
        return out
