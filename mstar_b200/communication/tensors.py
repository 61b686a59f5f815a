"""Tensor data plane. Every entity keeps its produced tensors in a ``TensorStore`` (uuid -> tensor, reference
counted, optionally persisted for the whole request). A ``TensorPointerInfo`` travels on the control mesh; the
consumer resolves it through its ``TensorCommunicationManager``:

  * same process  -> the producer's tensor itself (no copy);
  * other process, GPU tensor, same box -> CUDA IPC handle in the descriptor, the consumer maps the producer's
    allocation and peer-copies over NVLink into its own memory (no host bounce);
  * other process, host tensor (or IPC disabled) -> the C++ shared-memory arena, zero-copy view on the consumer.

Reference counterparts: ``TensorStore`` (mstar/communication/tensors.py:50-109), ``TensorCommunicationManager``
(:344-828), SHM-file / arena / Mooncake transports (:835-1246), CUDA-IPC KV transfer (mstar/engine/kv_store.py:
354-446).
"""
from __future__ import annotations

import threading
import uuid as _uuid

import torch

from ..graph.ir import TensorPointerInfo, fast_uid
from .arena import ShmArena, ShmArenaReader, dtype_from_name, dtype_name

# process-wide registry of stores, so that entities living in one process hand tensors over by reference
_PROCESS_STORES: dict[str, "TensorStore"] = {}
_PROCESS_LOCK = threading.Lock()


class TensorStore:
    def __init__(self, entity_id: str):
        self.entity_id = entity_id
        self._t: dict[str, torch.Tensor] = {}
        self._ref: dict[str, int] = {}
        self._persist: set[str] = set()
        self._by_request: dict[str, set[str]] = {}
        self._owner: dict[str, str] = {}
        self._lock = threading.Lock()

    def put(self, request_id: str, t: torch.Tensor, uuid: str | None = None, refs: int = 1, persist: bool = False) -> str:
        uuid = uuid or fast_uid()
        with self._lock:
            self._t[uuid] = t
            self._ref[uuid] = refs
            if persist:
                self._persist.add(uuid)
            self._by_request.setdefault(request_id, set()).add(uuid)
            self._owner[uuid] = request_id
        return uuid

    def get(self, uuid: str) -> torch.Tensor | None:
        return self._t.get(uuid)

    def increment_ref(self, uuid: str, n: int = 1) -> None:
        with self._lock:
            if uuid in self._ref:
                self._ref[uuid] += n

    def dereference(self, uuid: str, n: int = 1) -> bool:
        """Drop references; returns True when the tensor was released."""
        with self._lock:
            if uuid not in self._ref:
                return False
            self._ref[uuid] -= n
            if self._ref[uuid] <= 0 and uuid not in self._persist:
                self._drop(uuid)
                return True
        return False

    def adopt(self, uuid: str, owner: str, extra_refs: int = 1) -> bool:
        """Move a tensor to another owner and add references (a tensor that became a client result after it was
        stored as an intermediate must outlive the request's teardown)."""
        with self._lock:
            if uuid not in self._t:
                return False
            old = self._owner.get(uuid)
            if old is not None and old in self._by_request:
                self._by_request[old].discard(uuid)
            self._by_request.setdefault(owner, set()).add(uuid)
            self._owner[uuid] = owner
            self._ref[uuid] = max(0, self._ref.get(uuid, 0)) + extra_refs
            return True

    def owner_of(self, uuid: str) -> str | None:
        return self._owner.get(uuid)

    def unpersist(self, uuid: str) -> None:
        with self._lock:
            self._persist.discard(uuid)
            if self._ref.get(uuid, 1) <= 0:
                self._drop(uuid)

    def _drop(self, uuid: str) -> None:
        self._t.pop(uuid, None)
        self._ref.pop(uuid, None)
        self._persist.discard(uuid)
        owner = self._owner.pop(uuid, None)
        if owner is not None:
            s = self._by_request.get(owner)
            if s is not None:
                s.discard(uuid)

    def remove_request(self, request_id: str) -> int:
        with self._lock:
            ids = self._by_request.pop(request_id, set())
            for u in list(ids):
                self._t.pop(u, None)
                self._ref.pop(u, None)
                self._persist.discard(u)
                self._owner.pop(u, None)
            return len(ids)

    def __len__(self) -> int:
        return len(self._t)


class TensorCommunicationManager:
    def __init__(self, entity_id: str, device="cpu", *, arena_prefix: str | None = None, use_cuda_ipc: bool = True,
                 arena_segment_bytes: int = 256 << 20):
        self.entity_id = entity_id
        self.device = torch.device(device)
        self.store = TensorStore(entity_id)
        self.use_cuda_ipc = use_cuda_ipc
        self._arena_prefix = arena_prefix
        self._arena: ShmArena | None = None
        self._arena_lock = threading.Lock()
        self._arena_bytes = arena_segment_bytes
        self._reader: ShmArenaReader | None = None
        self.tx_bytes = 0
        self.rx_bytes = 0
        # per-transfer records feed the request profile; they are kept only while a profile is being collected
        # (log_transfers), never on the plain serving path, where they would grow with every chunk sent
        self.log_transfers = False
        self.tx_log: list[dict] = []
        self.rx_log: list[dict] = []
        with _PROCESS_LOCK:
            _PROCESS_STORES[entity_id] = self.store

    # ---- producer side ----
    def store_and_return_tensor_info(self, request_id: str, t: torch.Tensor, refs: int = 1, persist: bool = False,
                                     uuid: str | None = None) -> TensorPointerInfo:
        uuid = self.store.put(request_id, t, uuid=uuid, refs=refs, persist=persist)
        return TensorPointerInfo(dims=list(t.shape), dtype=dtype_name(t.dtype), nbytes=t.numel() * t.element_size(),
                                 address=t.data_ptr() if t.numel() else 0, stride=list(t.stride()), uuid=uuid,
                                 source_entity=self.entity_id,
                                 device_index=t.device.index if t.is_cuda else -1)

    def is_local(self, entity: str) -> bool:
        """True when ``entity``'s tensor store lives in this process (its descriptors resolve without a transport)."""
        return entity in _PROCESS_STORES

    def prepare_for_remote(self, info: TensorPointerInfo, dst_entity: str) -> TensorPointerInfo:
        """Make a descriptor resolvable by ``dst_entity``. In-process consumers need nothing; others get a CUDA
        IPC handle (GPU tensors) or an arena block (host tensors)."""
        if dst_entity in _PROCESS_STORES:
            return info
        t = self.store.get(info.uuid)
        if t is None:
            return info
        out = info.clone()
        if t.is_cuda and self.use_cuda_ipc:
            tc = t.contiguous()
            if tc is not t:
                self.store._t[info.uuid] = tc
            st = tc.untyped_storage()
            out.shm_segment = "cuda_ipc"
            out.cuda_ipc = (st._share_cuda_(), tc.storage_offset())      # type: ignore[attr-defined]
            out.stride = list(tc.stride())
        else:
            with self._arena_lock:      # two preprocess threads may send their first tensors at the same moment
                if self._arena is None:
                    prefix = self._arena_prefix or "mstar"
                    self._arena = ShmArena(f"{prefix}.{self.entity_id}.arena", segment_bytes=self._arena_bytes)
                    if self.device.type == "cuda":       # device-to-host writes into the arena become plain DMA
                        self._arena.pin()
                seg, off = self._arena.write(info.uuid, t)
            out.shm_segment = f"{self._arena.base_name}#{seg}"
            out.shm_offset = off
        self.tx_bytes += info.nbytes
        if self.log_transfers:
            self.tx_log.append(dict(uuid=info.uuid, nbytes=info.nbytes, dst=dst_entity))
        return out

    # ---- consumer side ----
    def read(self, info: TensorPointerInfo, device=None) -> torch.Tensor:
        device = torch.device(device) if device is not None else self.device
        src_store = _PROCESS_STORES.get(info.source_entity)
        t = src_store.get(info.uuid) if src_store is not None else None
        if t is None:
            if info.shm_segment == "cuda_ipc":
                t = self._read_cuda_ipc(info)
            elif info.shm_segment:
                base, seg = info.shm_segment.rsplit("#", 1)
                with self._arena_lock:
                    if self._reader is None:
                        self._reader = ShmArenaReader(pin=self.device.type == "cuda")
                    t = self._reader.view(base, int(seg), info.shm_offset, info.nbytes, dtype_from_name(info.dtype),
                                          info.dims).clone()
            else:
                raise KeyError(f"tensor {info.uuid} from {info.source_entity} is not reachable from {self.entity_id}")
            self.rx_bytes += info.nbytes
            if self.log_transfers:
                self.rx_log.append(dict(uuid=info.uuid, nbytes=info.nbytes, src=info.source_entity))
        if info.offset or info.source_tp_size > 1:
            pass    # sharded reads are resolved by parallel.sharding before the descriptor reaches this point
        if t.device != device:
            t = t.to(device, non_blocking=True)      # GPU -> GPU: peer copy over NVLink
        return t

    def read_bytes(self, info: TensorPointerInfo) -> bytes:
        """The tensor's raw bytes (row-major), without building a tensor when it sits in a shared-memory block: what
        the API process needs from payloads that are already in their wire format (16-bit PCM)."""
        src_store = _PROCESS_STORES.get(info.source_entity)
        t = src_store.get(info.uuid) if src_store is not None else None
        if t is None and info.shm_segment and info.shm_segment != "cuda_ipc":
            base, seg = info.shm_segment.rsplit("#", 1)
            with self._arena_lock:
                if self._reader is None:
                    self._reader = ShmArenaReader(pin=self.device.type == "cuda")
                reader = self._reader
            self.rx_bytes += info.nbytes
            return reader.read_bytes(base, int(seg), info.shm_offset, info.nbytes)
        if t is None:
            t = self.read(info, "cpu")
        return t.detach().cpu().contiguous().numpy().tobytes()

    def _read_cuda_ipc(self, info: TensorPointerInfo) -> torch.Tensor:
        from torch.multiprocessing.reductions import rebuild_cuda_tensor
        handle, storage_offset = info.cuda_ipc      # type: ignore[attr-defined]
        (dev, ipc_handle, size_bytes, off_bytes, ref_handle, ref_off, ev_handle, ev_sync) = handle
        return rebuild_cuda_tensor(torch.Tensor, tuple(info.dims), tuple(info.stride), storage_offset,
                                   torch.UntypedStorage, dtype_from_name(info.dtype), dev, ipc_handle, size_bytes,
                                   off_bytes, ref_handle, ref_off, ev_handle, ev_sync, requires_grad=False)

    # ---- lifetime ----
    def dereference(self, request_id: str, uuid: str, n: int = 1) -> None:
        if self.store.dereference(uuid, n) and self._arena is not None:
            self._arena.free(uuid)

    def increment_ref(self, request_id: str, uuid: str, n: int = 1) -> None:
        self.store.increment_ref(uuid, n)

    def remove_request(self, request_id: str) -> None:
        self.store.remove_request(request_id)

    def close(self) -> None:
        with _PROCESS_LOCK:
            _PROCESS_STORES.pop(self.entity_id, None)
        if self._arena is not None:
            self._arena.close()
        if self._reader is not None:
            self._reader.close()
