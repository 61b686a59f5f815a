"""Python side of the native HTTP frontend: starts the ``mstar-server`` binary and answers its requests.

Every request frame that arrives on the ``api_bridge`` mailbox is run through the SAME ASGI application that
uvicorn would serve (``create_app``), so all routes — ``/generate``, the OpenAI-compatible ``/v1/*``, ``/metrics``
— behave identically behind either frontend; response body parts are forwarded to the binary as they are produced,
which gives streaming (NDJSON / SSE) for free. A client that disconnects makes the binary send an ABORT frame;
the bridge cancels the ASGI task, which aborts the request in the engine.

Reference counterpart: the ``--rust-frontend`` mode of mstar/api_server/entrypoint.py:888-905 and its bridge
directory protocol.
"""
from __future__ import annotations

import asyncio
import ctypes
import json
import os
import struct
import subprocess
import threading
import time
import uuid

from ..ops import _lib

LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")


class _RawMesh:
    """Byte-frame mailbox (no pickling: the peer is the C++ binary)."""

    def __init__(self, prefix: str, entity: str, ring_bytes: int = 64 << 20):
        L = self.lib = _lib.runtime()
        L.mstar_mesh_create.restype = ctypes.c_void_p
        L.mstar_mesh_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_ulonglong]
        L.mstar_mesh_send.restype = ctypes.c_int
        L.mstar_mesh_send.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_ulonglong]
        L.mstar_mesh_recv.restype = ctypes.c_longlong
        L.mstar_mesh_recv.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_int]
        L.mstar_mesh_peek_size.restype = ctypes.c_longlong
        L.mstar_mesh_peek_size.argtypes = [ctypes.c_void_p]
        L.mstar_mesh_destroy.argtypes = [ctypes.c_void_p, ctypes.c_int]
        self.h = L.mstar_mesh_create(prefix.encode(), entity.encode(), ring_bytes)
        if not self.h:
            raise RuntimeError(f"cannot create mailbox {prefix}/{entity}")
        self._buf = ctypes.create_string_buffer(4 << 20)
        self._lock = threading.Lock()

    def send(self, dst: str, data: bytes, timeout_s: float = 10.0) -> bool:
        deadline = time.time() + timeout_s
        while True:
            with self._lock:
                rc = self.lib.mstar_mesh_send(self.h, dst.encode(), data, len(data))
            if rc == 0:
                return True
            if rc == -2 and time.time() < deadline:
                time.sleep(0.001)
                continue
            return False

    def recv(self, timeout_ms: int) -> bytes | None:
        n = self.lib.mstar_mesh_recv(self.h, self._buf, len(self._buf), timeout_ms)
        if n == -3:
            need = self.lib.mstar_mesh_peek_size(self.h)
            self._buf = ctypes.create_string_buffer(int(max(need, 2 * len(self._buf))))
            n = self.lib.mstar_mesh_recv(self.h, self._buf, len(self._buf), 0)
        return ctypes.string_at(self._buf, n) if n > 0 else None

    def close(self):
        if self.h:
            self.lib.mstar_mesh_destroy(self.h, 1)
            self.h = None


class NativeFrontend:
    def __init__(self, app, host: str = "0.0.0.0", port: int = 8000, binary: str | None = None,
                 max_connections: int = 1024):
        self.app, self.host, self.port = app, host, port
        self.binary = binary or os.environ.get("MSTAR_SERVER_BIN") or os.path.join(LIB_DIR, "mstar-server")
        if not os.path.exists(self.binary):
            raise FileNotFoundError(f"{self.binary} is missing: run python -m mstar_b200.build")
        self.prefix = f"mstarfe{os.getpid()}{uuid.uuid4().hex[:6]}"
        self.mesh = _RawMesh(self.prefix, "api_bridge")
        self.max_connections = max_connections
        self.proc: subprocess.Popen | None = None
        self.loop = asyncio.new_event_loop()
        self.tasks: dict[int, asyncio.Task] = {}
        self.running = False
        self.stats = dict(requests=0, aborted=0, batches=0, batched_chunks=0)
        # body chunks whose binary field the frontend encodes: collected while the API server handles one message of a
        # worker (the chunks of all requests of a batch) and sent as one frame when it is done with the message
        self._batch: list[bytes] = []
        self._batch_n = 0
        self._batch_lock = threading.Lock()
        self._batching = False
        self._fast_routes = os.environ.get("MSTAR_FRONTEND_FAST_ROUTES", "1") != "0"

    # ---- life cycle ----
    BATCH_MAX = 256

    def _flush_batch(self) -> None:
        if not self._batch_n:
            return
        with self._batch_lock:             # the send stays inside: frames of two flushes must not swap
            if not self._batch_n:
                return
            n, pieces = self._batch_n, self._batch
            self._batch, self._batch_n = [], 0
            self.stats["batches"] += 1
            self.stats["batched_chunks"] += n
            self.mesh.send("frontend", b'{"kind":"b64_batch","n":%d}\n' % n + b"".join(pieces))

    def start(self, wait_s: float = 10.0) -> "NativeFrontend":
        server = getattr(getattr(self.app, "state", None), "mstar_server", None)
        if server is not None and hasattr(server, "after_message_hooks") and os.environ.get("MSTAR_FRONTEND_BATCH", "1") != "0":
            server.after_message_hooks.append(self._flush_batch)
            self._batching = True
        self.proc = subprocess.Popen([self.binary, "--prefix", self.prefix, "--host", self.host, "--port", str(self.port),
                                      "--max-connections", str(self.max_connections)])
        self.running = True
        threading.Thread(target=self._loop_thread, daemon=True, name="frontend-asgi").start()
        self._bridge = threading.Thread(target=self._recv_thread, daemon=True, name="frontend-bridge")
        self._bridge.start()
        deadline = time.time() + wait_s
        while time.time() < deadline:
            if self.proc.poll() is not None:
                raise RuntimeError(f"mstar-server exited with {self.proc.returncode}")
            if self.mesh.send("frontend", b'{"kind":"ready"}\n', timeout_s=0.2):
                return self
            time.sleep(0.05)
        raise RuntimeError("mstar-server did not open its mailbox")

    def stop(self) -> None:
        self.running = False
        if self.proc is not None and self.proc.poll() is None:
            self.mesh.send("frontend", b'{"kind":"shutdown"}\n', timeout_s=0.5)
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.terminate()
        self.loop.call_soon_threadsafe(self.loop.stop)
        # the bridge thread may be blocked inside the mailbox's receive: the mailbox is unmapped only after it left
        bridge = getattr(self, "_bridge", None)
        if bridge is not None and bridge is not threading.current_thread():
            bridge.join(2.0)
        if bridge is None or not bridge.is_alive():
            self.mesh.close()

    def wait(self) -> int:
        return self.proc.wait() if self.proc is not None else 0

    # ---- bridge ----
    def _loop_thread(self):
        asyncio.set_event_loop(self.loop)
        self.loop.run_forever()

    def _recv_thread(self):
        while self.running:
            frame = self.mesh.recv(100)
            if frame is None:
                continue
            nl = frame.find(b"\n")
            if nl < 0:
                continue
            try:
                hdr = json.loads(frame[:nl])
            except Exception:  # noqa: BLE001
                continue
            body = frame[nl + 1:nl + 1 + int(hdr.get("len", 0))]
            rid = int(hdr["id"])
            if hdr.get("method") == "ABORT":
                t = self.tasks.get(rid)
                if t is not None:
                    self.stats["aborted"] += 1
                    self.loop.call_soon_threadsafe(t.cancel)
                continue
            self.stats["requests"] += 1
            self.loop.call_soon_threadsafe(self._spawn, rid, hdr, body)      # one callback, one task per request

    def _spawn(self, rid: int, hdr: dict, body: bytes) -> None:
        task = self.loop.create_task(self._serve(rid, hdr, body))
        self.tasks[rid] = task

        def done(t, rid=rid):
            self.tasks.pop(rid, None)
            if not t.cancelled():
                t.exception()              # retrieved: failures were answered inside _serve
        task.add_done_callback(done)

    def _send(self, rid: int, kind: str, payload: bytes = b"", **extra) -> None:
        head = json.dumps({"id": rid, "kind": kind, **extra}, separators=(",", ":")).encode() + b"\n"
        self._flush_batch()                # a frame never overtakes chunks that were collected before it
        self.mesh.send("frontend", head + payload)

    def _direct(self, rid: int):
        """The body sink handed to a streaming response: ``push(piece)`` sends one chunk; ``push.b64(prefix, data,
        suffix)``, when present, queues the chunk prefix + base64(data) + suffix for the frontend to encode."""
        head = json.dumps({"id": rid, "kind": "chunk"}, separators=(",", ":")).encode() + b"\n"
        send = self.mesh.send

        def push(piece: bytes) -> None:
            if piece:
                self._flush_batch()
                send("frontend", head + piece)
        if self._batching:
            pack = struct.Struct("<QIII").pack

            def b64(prefix: bytes, data: bytes, suffix: bytes) -> None:
                with self._batch_lock:
                    self._batch += (pack(rid, len(prefix), len(data), len(suffix)), prefix, data, suffix)
                    self._batch_n += 1
                    full = self._batch_n >= self.BATCH_MAX
                if full:
                    self._flush_batch()
            push.b64, push.flush = b64, self._flush_batch
        return push

    async def _serve(self, rid: int, hdr: dict, body: bytes):
        headers = [(b"host", f"{self.host}:{self.port}".encode()), (b"content-length", str(len(body)).encode())]
        if hdr.get("content_type"):
            headers.append((b"content-type", hdr["content_type"].encode()))
        scope = {"type": "http", "asgi": {"version": "3.0"}, "http_version": "1.1", "method": hdr["method"],
                 "scheme": "http", "path": hdr["path"], "raw_path": hdr["path"].encode(),
                 "query_string": hdr.get("query", "").encode(), "headers": headers, "client": ("frontend", 0),
                 "server": (self.host, self.port), "root_path": "",
                 # body pieces may be pushed from any thread, straight to the frontend process
                 "extensions": {"mstar.direct_stream": self._direct(rid)}}
        sent_body = False
        disconnected = asyncio.Event()

        async def receive():
            nonlocal sent_body
            if not sent_body:
                sent_body = True
                return {"type": "http.request", "body": body, "more_body": False}
            await disconnected.wait()
            return {"type": "http.disconnect"}

        state = {"head": False}

        async def send(msg):
            if msg["type"] == "http.response.start":
                hd = {k.decode().lower(): v.decode() for k, v in msg.get("headers", [])}
                ctype = hd.get("content-type", "application/octet-stream")
                streaming = "content-length" not in hd
                state["head"] = True
                self._send(rid, "head", status=int(msg["status"]), content_type=ctype, streaming=streaming)
            elif msg["type"] == "http.response.body":
                if msg.get("body"):
                    self._send(rid, "chunk", bytes(msg["body"]))
                if not msg.get("more_body", False):
                    self._send(rid, "end")
        try:
            # routes that the application also offers without its framework layers (plain streaming /generate)
            fast = getattr(getattr(self.app, "state", None), "fast_routes", None) if self._fast_routes else None
            handler = fast.get((hdr["method"], hdr["path"])) if fast else None
            resp = handler(body, hdr.get("content_type", "")) if handler is not None else None
            if resp is not None:
                self.stats["fast"] = self.stats.get("fast", 0) + 1
                await resp(scope, receive, send)
            else:
                await self.app(scope, receive, send)
        except asyncio.CancelledError:
            disconnected.set()
            raise
        except Exception as e:  # noqa: BLE001
            if not state["head"]:
                self._send(rid, "head", status=500, content_type="application/json", streaming=False)
                self._send(rid, "chunk", json.dumps({"detail": f"{type(e).__name__}: {e}"}).encode())
            self._send(rid, "end")
