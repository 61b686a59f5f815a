"""Collective groups. ``CommGroup`` wraps a torch.distributed process group (NCCL on GPUs, gloo for CPU ranks)
behind a small API; ``CommGroup.trivial()`` is the size-1 no-op group. The NCCL calls here are the *baseline*
path and the bootstrap (handle exchange); the hot tensor-parallel paths use the fused kernels of
``mstar_b200.parallel.fused`` over the symmetric heap and only fall back to these collectives when the heap is
not available (CPU ranks, single process tests).

Reference counterparts: ``CommGroup`` (mstar/distributed/communication.py:8-162: all_gather :38-60, barrier :62-65,
all_reduce :67-71, reduce_scatter :73-104, broadcast :106-111, all_to_all :113-162), ``WorkerParallelGroups``
(:165-305), ``GlobalParallelConfig`` (:308-375).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


class CommGroup:
    def __init__(self, group=None, ranks: list[int] | None = None, rank: int = 0):
        self.group = group
        self.ranks = list(ranks) if ranks is not None else [0]
        self.global_rank = rank
        self.size = len(self.ranks)
        self.rank = self.ranks.index(rank) if rank in self.ranks else 0
        self.symm = None   # SymmetricHeap attached by parallel.symm when available
        self.instance = None   # group over all tp x sp ranks of the model instance (tensor-parallel index slowest)

    @classmethod
    def trivial(cls) -> "CommGroup":
        return cls(None, [0], 0)

    @property
    def is_trivial(self) -> bool:
        return self.size == 1

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.size == 1:
            return x
        x = x.contiguous()
        out = torch.empty((self.size * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=self.group)
        dim = dim % x.dim()
        return torch.cat(list(out.chunk(self.size, 0)), dim=dim) if dim != 0 else out

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.size == 1:
            return x
        if dim != 0:
            x = x.transpose(0, dim)
        x = x.contiguous()
        out = torch.empty((x.shape[0] // self.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x, group=self.group)
        else:       # gloo has no reduce-scatter
            full = x.clone()
            dist.all_reduce(full, group=self.group)
            out.copy_(full.chunk(self.size, 0)[self.rank])
        return out.transpose(0, dim) if dim != 0 else out

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.size > 1:
            dist.broadcast(x, src=self.ranks[src], group=self.group)
        return x

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    def all_to_all(self, x: torch.Tensor, in_splits: list[int] | None = None,
                   out_splits: list[int] | None = None) -> torch.Tensor:
        """Split dim 0 of ``x`` by ``in_splits`` over the ranks; receive ``out_splits`` rows from each rank."""
        if self.size == 1:
            return x
        x = x.contiguous()
        if in_splits is None:
            in_splits = [x.shape[0] // self.size] * self.size
        if out_splits is None:
            out_splits = in_splits
        out = torch.empty((sum(out_splits), *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x, out_splits, in_splits, group=self.group)
        return out


@dataclass
class GlobalParallelConfig:
    """Mesh layout of one node group: ranks form a row-major [sp][tp] grid."""
    ranks: list[int] = field(default_factory=lambda: [0])
    tp_size: int = 1
    sp_size: int = 1

    def __post_init__(self):
        if self.tp_size * self.sp_size not in (len(self.ranks), 1) and len(self.ranks) % (self.tp_size * self.sp_size):
            raise ValueError(f"{len(self.ranks)} ranks cannot form instances of tp {self.tp_size} x sp {self.sp_size}")

    @property
    def instance_size(self) -> int:
        return self.tp_size * self.sp_size

    def instances(self) -> list[list[int]]:
        n = self.instance_size
        return [self.ranks[i:i + n] for i in range(0, len(self.ranks), n)]

    def tp_groups(self) -> list[list[int]]:
        out = []
        for inst in self.instances():
            for s in range(self.sp_size):
                out.append(inst[s * self.tp_size:(s + 1) * self.tp_size])
        return out

    def sp_groups(self) -> list[list[int]]:
        out = []
        for inst in self.instances():
            for t in range(self.tp_size):
                out.append([inst[s * self.tp_size + t] for s in range(self.sp_size)])
        return out


class WorkerParallelGroups:
    """Process-group bootstrap of one worker: a world group plus every TP / SP sub-group of the deployment.
    ``dist.new_group`` is collective over the world, so every rank creates every group in the same order."""

    def __init__(self, rank: int, world_size: int):
        self.rank, self.world_size = rank, world_size
        self.world: CommGroup = CommGroup.trivial()
        self._groups: dict[tuple[int, ...], CommGroup] = {}
        self.initialized = False

    def init_dist(self, init_method: str, backend: str | None = None, timeout_s: float = 600.0,
                  all_rank_tuples: list[tuple[int, ...]] | None = None) -> None:
        if self.world_size <= 1:
            return
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if not dist.is_initialized():
            dist.init_process_group(backend, init_method=init_method, rank=self.rank, world_size=self.world_size,
                                    timeout=datetime.timedelta(seconds=timeout_s))
        self.initialized = True
        self.world = CommGroup(dist.group.WORLD, list(range(self.world_size)), self.rank)
        for tup in sorted(set(all_rank_tuples or [])):
            if len(tup) <= 1:
                continue
            g = dist.new_group(list(tup))
            if self.rank in tup:
                self._groups[tuple(tup)] = CommGroup(g, list(tup), self.rank)

    def group_for(self, ranks: list[int] | tuple[int, ...]) -> CommGroup:
        ranks = tuple(ranks)
        if len(ranks) <= 1:
            return CommGroup.trivial()
        if ranks == tuple(range(self.world_size)) and ranks not in self._groups:
            return self.world
        return self._groups[ranks]

    def barrier_all(self) -> None:
        self.world.barrier()

    def shutdown(self) -> None:
        if self.initialized and dist.is_initialized():
            dist.destroy_process_group()
            self.initialized = False


def init_from_env(backend: str | None = None) -> CommGroup:
    """World group from torchrun's environment (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world <= 1:
        return CommGroup.trivial()
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return CommGroup(dist.group.WORLD, list(range(world)), rank)
