"""Control mesh: every entity (API server, conductor, each worker) owns a mailbox; ``send`` never blocks on the
receiver, ``drain`` returns everything that arrived, ``recv_or_wake`` sleeps until a message or a wake-up.

Two implementations share the interface:
  * ``LocalCommunicator`` — in-process mailboxes (single-process serving, unit tests);
  * ``ShmMeshCommunicator`` — the C++ shared-memory mesh (``csrc/runtime/mesh.cpp``): one lock-free multi-producer
    ring per entity in /dev/shm with a futex-based wake-up, payloads pickled.

Reference counterparts: ZMQ PUSH/PULL communicator (mstar/communication/communicator.py:19-220), the Rust
``RawZmqCommunicator`` with GIL-released send/drain/recv_or_wake (rust/src/communicator.rs:99-305) and its Python
wrapper (mstar/communication/rust_communicator.py).
"""
from __future__ import annotations

import ctypes
import pickle
import queue
import threading
import time

from ..utils.ipc_format import Message


class BaseCommunicator:
    entity_id: str

    def send(self, dst: str, msg: Message) -> None:
        raise NotImplementedError

    def drain(self) -> list[Message]:
        raise NotImplementedError

    def recv_or_wake(self, timeout_s: float = 0.05) -> list[Message]:
        raise NotImplementedError

    def wake(self) -> None:
        pass

    def close(self) -> None:
        pass

    # reference-compatible spelling
    def get_all_new_messages(self) -> list[Message]:
        return self.drain()


class _LocalHub:
    def __init__(self):
        self.boxes: dict[str, queue.Queue] = {}
        self.lock = threading.Lock()

    def box(self, entity: str) -> queue.Queue:
        with self.lock:
            return self.boxes.setdefault(entity, queue.Queue())


class LocalCommunicator(BaseCommunicator):
    """Mailboxes inside one process; ``hub`` is shared by the communicators of all entities."""
    _default_hub = _LocalHub()

    def __init__(self, entity_id: str, hub: _LocalHub | None = None):
        self.entity_id = entity_id
        self.hub = hub or LocalCommunicator._default_hub
        self.inbox = self.hub.box(entity_id)
        self.sent: list[tuple[str, Message]] = []      # record for tests
        self.record = False

    @staticmethod
    def new_hub() -> _LocalHub:
        return _LocalHub()

    def send(self, dst: str, msg: Message) -> None:
        msg.src = msg.src or self.entity_id
        if self.record:
            self.sent.append((dst, msg))
        self.hub.box(dst).put(msg)

    def drain(self) -> list[Message]:
        out = []
        while True:
            try:
                m = self.inbox.get_nowait()
            except queue.Empty:
                return out
            if m is not None:
                out.append(m)

    def recv_or_wake(self, timeout_s: float = 0.05) -> list[Message]:
        try:
            first = self.inbox.get(timeout=timeout_s)
        except queue.Empty:
            return []
        rest = self.drain()
        return ([first] if first is not None else []) + rest

    def wake(self) -> None:
        self.inbox.put(None)


class ShmMeshCommunicator(BaseCommunicator):
    """Mailbox in shared memory, served by the C++ runtime library. ``prefix`` names the deployment (all entities
    of one server share it); every entity creates its own ring and opens its peers' rings lazily."""

    def __init__(self, entity_id: str, prefix: str, ring_bytes: int = 8 << 20):
        from ..ops import _lib
        self.lib = _lib.runtime()
        self.entity_id, self.prefix = entity_id, prefix
        L = self.lib
        L.mstar_mesh_create.restype = ctypes.c_void_p
        L.mstar_mesh_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_ulonglong]
        L.mstar_mesh_send.restype = ctypes.c_int
        L.mstar_mesh_send.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_ulonglong]
        L.mstar_mesh_recv.restype = ctypes.c_longlong
        L.mstar_mesh_recv.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_int]
        L.mstar_mesh_recv_us.restype = ctypes.c_longlong
        L.mstar_mesh_recv_us.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_longlong]
        L.mstar_mesh_peek_size.restype = ctypes.c_longlong
        L.mstar_mesh_peek_size.argtypes = [ctypes.c_void_p]
        L.mstar_mesh_wake.argtypes = [ctypes.c_void_p]
        L.mstar_mesh_destroy.argtypes = [ctypes.c_void_p, ctypes.c_int]
        self.h = L.mstar_mesh_create(prefix.encode(), entity_id.encode(), ring_bytes)
        if not self.h:
            raise RuntimeError(f"mesh: cannot create mailbox {prefix}/{entity_id}")
        self._buf = ctypes.create_string_buffer(1 << 20)
        self._send_lock = threading.Lock()

    def send(self, dst: str, msg: Message) -> None:
        msg.src = msg.src or self.entity_id
        data = pickle.dumps(msg, protocol=pickle.HIGHEST_PROTOCOL)
        deadline = time.time() + 10.0
        while True:
            with self._send_lock:
                rc = self.lib.mstar_mesh_send(self.h, dst.encode(), data, len(data))
            if rc == 0:
                return
            if rc == -2 and time.time() < deadline:      # ring full or peer not up yet: retry briefly
                time.sleep(0.001)
                continue
            raise RuntimeError(f"mesh: send to {dst} failed (rc={rc})")

    def _pop(self, timeout_us: int) -> Message | None:
        n = self.lib.mstar_mesh_recv_us(self.h, self._buf, len(self._buf), timeout_us)
        if n == -3:     # buffer too small
            need = self.lib.mstar_mesh_peek_size(self.h)
            self._buf = ctypes.create_string_buffer(int(max(need, len(self._buf) * 2)))
            n = self.lib.mstar_mesh_recv(self.h, self._buf, len(self._buf), 0)
        if n <= 0:
            return None
        return pickle.loads(ctypes.string_at(self._buf, n))

    def drain(self) -> list[Message]:
        out = []
        while True:
            m = self._pop(0)
            if m is None:
                return out
            out.append(m)

    def recv_or_wake(self, timeout_s: float = 0.05) -> list[Message]:
        m = self._pop(int(timeout_s * 1e6))
        return ([m] if m is not None else []) + self.drain()

    def wake(self) -> None:
        self.lib.mstar_mesh_wake(self.h)

    def close(self, unlink: bool = True) -> None:
        if self.h:
            self.lib.mstar_mesh_destroy(self.h, 1 if unlink else 0)
            self.h = None


def make_communicator(entity_id: str, kind: str = "local", prefix: str = "mstar", hub=None) -> BaseCommunicator:
    if kind == "local":
        return LocalCommunicator(entity_id, hub)
    if kind == "shm":
        return ShmMeshCommunicator(entity_id, prefix)
    raise ValueError(f"unknown communicator kind {kind!r}")
