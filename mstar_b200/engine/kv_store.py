"""Paged KV storage: page allocator, per-request/per-label page lists, host offload pool, peer transfer.

The pool of one engine is a list of per-layer tensors ``[num_pages, 2, Hkv, page_size, D]`` (zero-initialised:
the attention kernel may read masked slots, which therefore must hold finite values). A request owns pages per
*label* (``main``, ``cfg_text``, ``cfg_img``, ``uncond`` ...), so CFG branches keep separate contexts.

Reference counterparts: ``PageAllocator`` (mstar/engine/kv_store.py:25-67), ``KVCacheConfig`` (:102-145),
``KVRequestState`` (:155-181), ``AllocationFailedError`` (:187-208), ``PagedAllocationManager`` (:465-731),
``CPUPagePool`` (mstar/engine/cpu_page_pool.py), CUDA-IPC / Mooncake KV transfer engines (:264-446) — here KV
pages move between GPUs of the box with peer copies (``PeerKVTransfer``).
"""
from __future__ import annotations

import threading
from collections import deque
from dataclasses import dataclass, field, replace

import torch


class AllocationFailedError(RuntimeError):
    """Raised when the pool cannot serve a batch. Carries what is needed to pick an offload victim."""

    def __init__(self, requested: int, available: int, request_ids: list[str] | None = None):
        super().__init__(f"KV pool exhausted: need {requested} pages, {available} free")
        self.requested, self.available = requested, available
        self.request_ids = list(request_ids or [])


class PageAllocator:
    """FIFO free list, safe against concurrent allocate/free from the GPU thread and the plan thread."""

    def __init__(self, max_num_pages: int):
        self.max_num_pages = max_num_pages
        self._free: deque[int] = deque(range(max_num_pages))
        self._lock = threading.Lock()

    def try_allocate(self, n: int) -> list[int] | None:
        with self._lock:
            if len(self._free) < n:
                return None
            return [self._free.popleft() for _ in range(n)]

    def allocate(self, n: int) -> list[int]:
        pages = self.try_allocate(n)
        if pages is None:
            raise AllocationFailedError(n, self.num_free)
        return pages

    def free(self, pages: list[int]) -> None:
        with self._lock:
            self._free.extend(pages)

    @property
    def num_free(self) -> int:
        return len(self._free)


@dataclass(frozen=True)
class CrossAttnKVConfig:
    """A read-only context pool (encoder K/V written once, read by every decode step)."""
    name: str
    num_kv_heads: int
    head_dim: int
    max_context_len: int
    max_contexts: int = 64


@dataclass
class KVCacheConfig:
    num_layers: int
    num_kv_heads: int
    head_dim: int
    max_seq_len: int = 8192
    max_num_pages: int = 2048
    page_size: int = 128
    num_qo_heads: int = 0
    cpu_offload_pages: int = 0
    nodes: list[str] = field(default_factory=list)
    cross_attn: list[CrossAttnKVConfig] = field(default_factory=list)
    attention_backend: str = "tcgen05"      # accepted for config compatibility: "flashinfer" | "dense_gen"
    dtype: torch.dtype = torch.bfloat16

    def __post_init__(self):
        ps = self.page_size
        if ps < 8 or ps > 128 or ps & (ps - 1):
            raise ValueError("page_size must be a power of two in [8, 128]")

    def shard(self, num_shards: int) -> "KVCacheConfig":
        """Per-rank config under head sharding (TP x SP ranks each hold Hkv / shards heads; replicated if fewer)."""
        kv = max(1, self.num_kv_heads // num_shards)
        qo = max(1, self.num_qo_heads // num_shards) if self.num_qo_heads else 0
        return replace(self, num_kv_heads=kv, num_qo_heads=qo)

    def bytes_per_page(self) -> int:
        return 2 * self.num_kv_heads * self.page_size * self.head_dim * torch.finfo(self.dtype).bits // 8 * self.num_layers


@dataclass
class KVRequestState:
    pages: list[int] = field(default_factory=list)
    seq_len: int = 0                 # tokens whose K/V are in the pool
    pos_offset: int = 0              # rope position of the next token minus seq_len (custom position advance)
    offloaded: bool = False
    cpu_pages: list[int] = field(default_factory=list)

    def get_pos_info(self) -> tuple[int, int]:
        return self.seq_len, self.seq_len + self.pos_offset


class CPUPagePool:
    """Pinned host mirror for offloaded pages; copies run on a side stream."""

    def __init__(self, num_pages: int, layer_shapes: list[torch.Size], dtype: torch.dtype, pin: bool = True):
        self.allocator = PageAllocator(num_pages)
        pin = pin and torch.cuda.is_available()
        self.layers = [torch.zeros((num_pages, *s[1:]), dtype=dtype, pin_memory=pin) for s in layer_shapes]
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def offload(self, kv_layers: list[torch.Tensor], gpu_pages: list[int]) -> list[int]:
        cpu_pages = self.allocator.allocate(len(gpu_pages))
        gi = torch.tensor(gpu_pages, dtype=torch.long, device=kv_layers[0].device)
        if self.stream is not None and kv_layers[0].is_cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                for host, dev in zip(self.layers, kv_layers):
                    host[cpu_pages] = dev[gi].to("cpu", non_blocking=False)
            self.stream.synchronize()
        else:
            for host, dev in zip(self.layers, kv_layers):
                host[cpu_pages] = dev[gi].cpu()
        return cpu_pages

    def reload(self, kv_layers: list[torch.Tensor], cpu_pages: list[int], gpu_pages: list[int]) -> None:
        gi = torch.tensor(gpu_pages, dtype=torch.long, device=kv_layers[0].device)
        for host, dev in zip(self.layers, kv_layers):
            dev[gi] = host[cpu_pages].to(dev.device, non_blocking=True)
        self.allocator.free(cpu_pages)


class PagedAllocationManager:
    """Owns the page pool of one engine and the per-(request, label) page lists."""

    def __init__(self, config: KVCacheConfig, device, allocate_storage: bool = True):
        self.config = config
        self.device = torch.device(device)
        self.allocator = PageAllocator(config.max_num_pages)
        self._lock = threading.RLock()
        self._states: dict[str, dict[str, KVRequestState]] = {}
        self.kv_layers: list[torch.Tensor] = []
        if allocate_storage:
            shape = (config.max_num_pages, 2, config.num_kv_heads, config.page_size, config.head_dim)
            self.kv_layers = [torch.zeros(shape, dtype=config.dtype, device=self.device)
                              for _ in range(config.num_layers)]
        self.cpu_pool: CPUPagePool | None = None
        if config.cpu_offload_pages > 0 and allocate_storage:
            self.cpu_pool = CPUPagePool(config.cpu_offload_pages, [l.shape for l in self.kv_layers], config.dtype)

    # ---- bookkeeping ----
    @property
    def num_free_pages(self) -> int:
        return self.allocator.num_free

    @property
    def total_pages(self) -> int:
        return self.config.max_num_pages

    def add_request(self, request_id: str, labels: list[str] | None = None) -> None:
        with self._lock:
            st = self._states.setdefault(request_id, {})
            for lb in labels or ["main"]:
                st.setdefault(lb, KVRequestState())

    def has_request(self, request_id: str) -> bool:
        return request_id in self._states

    def get_state(self, request_id: str, label: str = "main") -> KVRequestState:
        with self._lock:
            return self._states.setdefault(request_id, {}).setdefault(label, KVRequestState())

    def get_labels(self, request_id: str) -> list[str]:
        return list(self._states.get(request_id, {}))

    def get_per_label_seq_info(self, request_id: str) -> dict[str, tuple[int, int]]:
        return {lb: st.get_pos_info() for lb, st in self._states.get(request_id, {}).items()}

    def pages_of(self, request_id: str) -> int:
        return sum(len(s.pages) for s in self._states.get(request_id, {}).values())

    # ---- allocation ----
    def pages_needed(self, request_id: str, label: str, new_tokens: int) -> int:
        st = self.get_state(request_id, label)
        ps = self.config.page_size
        return max(0, (st.seq_len + new_tokens + ps - 1) // ps - len(st.pages))

    def alloc(self, request_id: str, label: str, new_tokens: int) -> KVRequestState:
        """Make room for ``new_tokens`` more tokens. Raises AllocationFailedError and leaves state untouched."""
        with self._lock:
            st = self.get_state(request_id, label)
            need = self.pages_needed(request_id, label, new_tokens)
            if need:
                pages = self.allocator.try_allocate(need)
                if pages is None:
                    raise AllocationFailedError(need, self.allocator.num_free, [request_id])
                st.pages.extend(pages)
            return st

    def alloc_batch(self, items: list[tuple[str, str, int]]) -> None:
        """All-or-nothing allocation for a batch of (request, label, new_tokens)."""
        with self._lock:
            needs = [self.pages_needed(r, lb, n) for r, lb, n in items]
            total = sum(needs)
            if total > self.allocator.num_free:
                raise AllocationFailedError(total, self.allocator.num_free, [r for r, _, _ in items])
            for (r, lb, _), n in zip(items, needs):
                if n:
                    self.get_state(r, lb).pages.extend(self.allocator.allocate(n))

    def reset_label(self, request_id: str, label: str, free: bool = True) -> None:
        with self._lock:
            st = self._states.get(request_id, {}).get(label)
            if st is None:
                return
            if free and st.pages:
                self.allocator.free(st.pages)
            st.pages, st.seq_len, st.pos_offset = [], 0, 0

    def export_descriptor(self, request_id: str) -> dict:
        """What a peer pool needs to pull this request's K/V: per label the page ids, length and position offset."""
        with self._lock:
            return {lb: dict(pages=list(st.pages), seq_len=st.seq_len, pos_offset=st.pos_offset)
                    for lb, st in self._states.get(request_id, {}).items()}

    def copy_label(self, request_id: str, src: str, dst: str) -> None:
        """Snapshot: ``dst`` gets its own copy of ``src``'s pages (page copy on the device)."""
        with self._lock:
            s = self.get_state(request_id, src)
            self.reset_label(request_id, dst)
            d = self.get_state(request_id, dst)
            if s.pages:
                d.pages = self.allocator.allocate(len(s.pages))
                si = torch.tensor(s.pages, dtype=torch.long, device=self.device)
                di = torch.tensor(d.pages, dtype=torch.long, device=self.device)
                for layer in self.kv_layers:
                    layer[di] = layer[si]
            d.seq_len, d.pos_offset = s.seq_len, s.pos_offset

    def remove_request(self, request_id: str) -> None:
        with self._lock:
            st = self._states.pop(request_id, None)
            if not st:
                return
            for s in st.values():
                if s.pages:
                    self.allocator.free(s.pages)
                if s.cpu_pages and self.cpu_pool is not None:
                    self.cpu_pool.allocator.free(s.cpu_pages)

    def cleanup(self) -> None:
        for rid in list(self._states):
            self.remove_request(rid)

    # ---- offload / reload ----
    def offload_request(self, request_id: str) -> int:
        """Move all pages of a request to the host pool; returns the number of device pages freed."""
        if self.cpu_pool is None:
            return 0
        freed = 0
        with self._lock:
            for st in self._states.get(request_id, {}).values():
                if st.offloaded or not st.pages:
                    continue
                st.cpu_pages = self.cpu_pool.offload(self.kv_layers, st.pages)
                self.allocator.free(st.pages)
                freed += len(st.pages)
                st.pages, st.offloaded = [], True
        return freed

    def is_offloaded(self, request_id: str) -> bool:
        return any(s.offloaded for s in self._states.get(request_id, {}).values())

    def reload_request(self, request_id: str) -> None:
        with self._lock:
            for st in self._states.get(request_id, {}).values():
                if not st.offloaded:
                    continue
                pages = self.allocator.try_allocate(len(st.cpu_pages))
                if pages is None:
                    raise AllocationFailedError(len(st.cpu_pages), self.allocator.num_free, [request_id])
                self.cpu_pool.reload(self.kv_layers, st.cpu_pages, pages)
                st.pages, st.cpu_pages, st.offloaded = pages, [], False

    # ---- transfer between engines (prefill/decode disaggregation) ----
    def export_request(self, request_id: str) -> dict:
        """Descriptor of a request's KV for a peer engine: page ids per label plus lengths."""
        return {lb: dict(pages=list(s.pages), seq_len=s.seq_len, pos_offset=s.pos_offset)
                for lb, s in self._states.get(request_id, {}).items()}


class PeerKVTransfer:
    """Copies a request's KV pages from a source pool (possibly on another GPU of the box) into this pool.
    Device-to-device copies go over NVLink when peer access is available; no host bounce."""

    def __init__(self, dst: PagedAllocationManager):
        self.dst = dst

    def pull(self, request_id: str, src_layers: list[torch.Tensor], descriptor: dict) -> None:
        for label, d in descriptor.items():
            self.dst.reset_label(request_id, label)
            st = self.dst.get_state(request_id, label)
            n = len(d["pages"])
            if n:
                st.pages = self.dst.allocator.allocate(n)
                di = torch.tensor(st.pages, dtype=torch.long, device=self.dst.device)
                for dl, sl in zip(self.dst.kv_layers, src_layers):
                    si = torch.tensor(d["pages"], dtype=torch.long, device=sl.device)
                    dl[di] = sl[si].to(dl.device, non_blocking=True)
            st.seq_len, st.pos_offset = d["seq_len"], d["pos_offset"]
