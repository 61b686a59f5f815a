"""API server core: request registry, preprocessing (media loading + ``model.process_prompt``) on a worker thread
pool, hand-off to the conductor, and delivery of result chunks back to waiting clients.

Reference counterparts: ``APIServer`` (mstar/api_server/entrypoint.py:158-674: submit :251-305, result loop
:359-577, TTL pruning, abort :652-668), ``PreprocessWorkerThread`` (mstar/api_server/data_worker.py:225-580).
"""
from __future__ import annotations

import logging
import queue
import threading
import time
import uuid
from concurrent.futures import ThreadPoolExecutor

import torch

from ..communication.tensors import TensorCommunicationManager
from ..conductor.deployment import Deployment
from ..utils import ipc_format as ipc
from ..utils.ipc_format import ApiMessageType as AM
from ..utils.ipc_format import ConductorMessageType as CM
from ..utils.ipc_format import Message
from .request_types import PendingRequest, ResultChunk

log = logging.getLogger("mstar.api")

_EXT_MODALITY = {".png": "image", ".jpg": "image", ".jpeg": "image", ".webp": "image", ".bmp": "image",
                 ".wav": "audio", ".mp3": "audio", ".flac": "audio", ".ogg": "audio",
                 ".mp4": "video", ".mov": "video", ".avi": "video", ".mkv": "video"}


def modality_of(filename: str) -> str | None:
    import os
    return _EXT_MODALITY.get(os.path.splitext(filename)[1].lower())


class APIServer:
    def __init__(self, config, *, in_process: bool = True, request_timeout_s: float = 600.0, result_ttl_s: float = 300.0,
                 log_stats: bool = False, log_stats_file: str | None = None, **deploy_kw):
        if log_stats or log_stats_file:
            from ..conductor.deployment import load_config
            config = dict(load_config(config), log_stats=True)     # workers collect per-request profiles
        self.log_stats_file = log_stats_file
        self.deployment = Deployment(config, in_process=in_process, **deploy_kw)
        self.model = self.deployment.model
        self.comm = self.deployment.api_comm
        self.tensors = TensorCommunicationManager("api", "cpu", arena_prefix=self.deployment.prefix)
        self.pending: dict[str, PendingRequest] = {}
        self.lock = threading.Lock()
        self.ready = threading.Event()
        self.request_timeout_s, self.result_ttl_s = request_timeout_s, result_ttl_s
        self.log_stats = bool(log_stats or log_stats_file)
        self.pre_pool = ThreadPoolExecutor(4, thread_name_prefix="preprocess")
        self.running = True
        self.stats = dict(submitted=0, completed=0, failed=0, aborted=0)
        self.after_message_hooks: list = []        # called on the result thread after every handled message
        # modality -> dtype name of client-bound tensors whose bytes ARE the payload (the model's ``postprocess`` would
        # only copy them out): 16-bit PCM quantised by the codec
        self._raw_payload: dict[str, str] = dict(getattr(self.model, "raw_payload_dtypes", None) or {})
        self._thread = threading.Thread(target=self._process_messages, daemon=True, name="api-results")

    # ---- lifecycle ----
    def start(self, wait_ready_s: float = 600.0) -> "APIServer":
        self.deployment.start()
        self._thread.start()
        deadline = time.time() + wait_ready_s
        while not self.ready.wait(0.5):
            dead = [p for p in self.deployment.procs if p.exitcode is not None]
            if dead:        # a conductor / worker process that ended during start-up never reports ready
                codes = [p.exitcode for p in dead]
                self.shutdown()
                raise RuntimeError(f"{len(dead)} deployment process(es) ended during start-up (exit codes {codes}); "
                                   "their log output above says why")
            if time.time() > deadline:
                raise TimeoutError("workers did not come up")
        return self

    def shutdown(self) -> None:
        self.running = False
        # the result thread may be blocked inside the mailbox's receive (50 ms slices): let it leave before the
        # deployment closes and unmaps that mailbox
        if self._thread.is_alive() and self._thread is not threading.current_thread():
            self._thread.join(2.0)
        self.deployment.shutdown()
        self.pre_pool.shutdown(wait=False)
        self.tensors.close()

    # ---- submission ----
    def submit_request(self, text: str | None = None, files: list[tuple[str, bytes]] | None = None,
                       input_modalities: list[str] | None = None, output_modalities: list[str] | None = None,
                       model_kwargs: dict | None = None, request_id: str | None = None,
                       tensors: dict | None = None) -> str:
        rid = request_id or uuid.uuid4().hex
        out_mod = output_modalities or ["text"]
        pr = PendingRequest(rid, out_mod, dict(model_kwargs or {}))
        with self.lock:
            self.pending[rid] = pr
        self.stats["submitted"] += 1
        self.pre_pool.submit(self._preprocess, pr, text, files or [], input_modalities, tensors or {})
        return rid

    def _preprocess(self, pr: PendingRequest, text, files, input_modalities, tensors) -> None:
        try:
            named: dict[str, list[torch.Tensor]] = {k: list(v) for k, v in tensors.items()}
            mods = list(input_modalities or (["text"] if text else []))
            for fname, blob in files:
                m = modality_of(fname)
                if m is None:
                    raise ValueError(f"cannot infer the modality of {fname!r}")
                loader = {"image": self.model.load_image, "audio": self.model.load_audio, "video": self.model.load_video}[m]
                named.setdefault(m, []).append(loader(blob))
                if m not in mods:
                    mods.append(m)
            sigs = self.model.process_prompt(text, mods, pr.output_modalities, named, **pr.model_kwargs)
            if text:
                pr.inputs["text"] = [1, len(text.encode())]
            for fname, blob in files:
                rec = pr.inputs.setdefault(modality_of(fname) or "file", [0, 0])
                rec[0] += 1
                rec[1] += len(blob)
            pr.t_preprocessed = time.time()
            infos = {k: [self.tensors.prepare_for_remote(self.tensors.store_and_return_tensor_info(pr.request_id, t, persist=True), "conductor_workers")
                         for t in v] for k, v in sigs.items()}
            body = ipc.NewRequestConductor(pr.request_id, infos, mods, pr.output_modalities, {}, pr.model_kwargs)
            self.comm.send("conductor", Message(CM.NEW_REQUEST, body))
        except Exception as e:  # noqa: BLE001
            log.exception("preprocess of %s failed", pr.request_id)
            self._finish(pr, ResultChunk("error", f"{type(e).__name__}: {e}".encode(), final=True, error_status=400))

    def abort_request(self, request_id: str) -> None:
        with self.lock:
            pr = self.pending.get(request_id)
        if pr is None or pr.done:
            return
        self.stats["aborted"] += 1
        self.comm.send("conductor", Message(CM.ABORT_REQUEST, ipc.AbortRequest(request_id)))
        self._finish(pr, ResultChunk("error", b"aborted", final=True, error_status=499))

    # ---- results ----
    @staticmethod
    def _put(pr: PendingRequest, chunk: ResultChunk) -> None:
        with pr.lock:
            if pr.sink is not None:     # a transport took this request over: no queue, no thread hop
                pr.sink(chunk)
                return
            pr.chunks.put(chunk)
        wake = pr.wake                  # set by an event-loop consumer that found the queue empty
        if wake is not None:
            pr.wake = None
            wake()

    def attach_sink(self, request_id: str, sink) -> None:
        """From now on every chunk of the request (the terminal one included) is handed to ``sink`` on the thread
        that produced it, in order, after whatever was already queued. ``sink`` must not block for long."""
        with self.lock:
            pr = self.pending.get(request_id)
        if pr is None:
            raise KeyError(request_id)
        with pr.lock:
            while True:
                try:
                    sink(pr.chunks.get_nowait())
                except queue.Empty:
                    break
            pr.sink = sink

    def detach_sink(self, request_id: str) -> None:
        with self.lock:
            pr = self.pending.get(request_id)
        if pr is not None:
            with pr.lock:
                pr.sink = None

    def _finish(self, pr: PendingRequest, last: ResultChunk | None = None) -> None:
        if pr.done:
            return
        pr.done = True
        self._put(pr, last or ResultChunk("done", final=True))
        self.tensors.remove_request(pr.request_id)

    def _process_messages(self) -> None:
        last_prune = time.time()
        while self.running:
            for m in self.comm.recv_or_wake(0.05):
                try:
                    self._handle(m)
                except Exception:  # noqa: BLE001
                    log.exception("api: message %s failed", m.type)
                for hook in self.after_message_hooks:      # transports that collect a message's chunks send them now
                    try:
                        hook()
                    except Exception:  # noqa: BLE001
                        log.exception("api: after-message hook failed")
            if time.time() - last_prune > 5.0:
                last_prune = time.time()
                self._prune()

    def _handle(self, m: Message) -> None:
        if m.type == AM.SETUP_DONE:
            self.ready.set()
            return
        if m.type == AM.RESULT_TENSORS_BATCH:
            acks: dict[str, list] = {}
            try:
                for rt in m.body.items:
                    try:
                        self._handle_result(rt, acks)
                    except Exception:  # noqa: BLE001
                        log.exception("api: result of %s failed", rt.request_id)
            finally:
                for src, items in acks.items():
                    self.comm.send(src, Message(ipc.WorkerMessageType.TENSOR_RECEIVED_BATCH,
                                                ipc.TensorReceivedBatch(items)))
            return
        b = m.body
        with self.lock:
            pr = self.pending.get(b.request_id)
        if m.type == AM.RESULT_TENSORS:
            acks = {}
            try:
                self._handle_result(b, acks)
            finally:
                for src, items in acks.items():
                    self.comm.send(src, Message(ipc.WorkerMessageType.TENSOR_RECEIVED, items[0]))
            return
        if pr is None or pr.done:
            return
        if m.type == AM.REQUEST_COMPLETE:
            pr.profile = b.profile
            self.stats["completed"] += 1
            if self.log_stats:
                from ..profile.display import render, write_profile
                write_profile(render(self.request_profile(pr)), self.log_stats_file)
            self._finish(pr)
        elif m.type == AM.REQUEST_FAILED:
            self.stats["failed"] += 1
            self._finish(pr, ResultChunk("error", b.error_message.encode(), final=True, error_status=b.status))

    def _handle_result(self, b, acks: dict) -> None:
        """One request's client-bound tensors: read, convert with the model's ``postprocess``, hand to the client.
        The acknowledgement that lets the producer free them is collected in ``acks`` (also when nobody waits)."""
        if b.source_entity:
            acks.setdefault(b.source_entity, []).append(
                ipc.TensorReceived(b.request_id + "#emit", {ti.uuid: 1 for ti in b.tensors}))
        with self.lock:
            pr = self.pending.get(b.request_id)
        if pr is None or pr.done:
            return
        if len(b.tensors) == 1 and self._raw_payload.get(b.modality) == b.tensors[0].dtype:
            data = self.tensors.read_bytes(b.tensors[0])       # already in its wire format: bytes straight from the block
        else:
            ts = [self.tensors.read(ti, "cpu") for ti in b.tensors]
            data = self.model.postprocess(ts[0] if len(ts) == 1 else ts, b.modality, pr.model_kwargs)
        pr.t_last_chunk = time.time()
        if pr.t_first_chunk is None:
            pr.t_first_chunk = pr.t_last_chunk
        rec = pr.outputs.setdefault(b.modality, [0, 0])
        rec[0] += 1
        rec[1] += len(data) if isinstance(data, (bytes, bytearray)) else 0
        self._put(pr, ResultChunk(b.modality, data, dict(b.metadata)))

    def request_profile(self, pr: PendingRequest):
        """The whole-request profile: this server's own timestamps and byte counts, the conductor's admission and
        completion times, and the node timings and transfers that the workers reported with every finished walk."""
        from ..profile.records import RequestProfile
        rp = RequestProfile(pr.request_id, inputs=dict(pr.inputs), outputs=dict(pr.outputs),
                            tokens_out=int(pr.profile.get("tokens_out", 0)))
        t0 = pr.t_submit
        pre = (pr.t_preprocessed - t0) if pr.t_preprocessed else None
        cp = {"received": 0.0, "preprocessed": pre,
              "first_chunk": (pr.t_first_chunk - t0) if pr.t_first_chunk else None,
              "last_chunk": (pr.t_last_chunk - t0) if pr.t_last_chunk else None, "finished": time.time() - t0}
        if pre is not None and "queue_s" in pr.profile:       # the conductor's clock starts when the request reaches it
            cp["admitted"] = pre + pr.profile["queue_s"]
            cp["conductor_done"] = pre + pr.profile.get("total_s", 0.0)
        rp.checkpoints = cp
        for w in pr.profile.get("walks", []):
            if isinstance(w, dict) and w.get("profile"):
                rp.merge_worker(w["profile"])
        return rp

    def _prune(self) -> None:
        now = time.time()
        with self.lock:
            for rid, pr in list(self.pending.items()):
                if pr.done and now - pr.t_submit > self.result_ttl_s:
                    del self.pending[rid]
                elif not pr.done and now - pr.t_submit > self.request_timeout_s:
                    self.comm.send("conductor", Message(CM.ABORT_REQUEST, ipc.AbortRequest(rid)))
                    self._finish(pr, ResultChunk("error", b"request timed out", final=True, error_status=500))

    def iter_result_chunks(self, request_id: str, timeout_s: float | None = None):
        with self.lock:
            pr = self.pending.get(request_id)
        if pr is None:
            raise KeyError(request_id)
        deadline = time.time() + (timeout_s or self.request_timeout_s)
        while True:
            try:
                c = pr.chunks.get(timeout=max(0.01, min(1.0, deadline - time.time())))
            except queue.Empty:
                if time.time() > deadline:
                    self.abort_request(request_id)
                    yield ResultChunk("error", b"request timed out", final=True, error_status=500)
                    return
                continue
            if c.modality == "done":
                return
            yield c
            if c.final:
                return

    async def aiter_result_chunks(self, request_id: str, timeout_s: float | None = None):
        """``iter_result_chunks`` for an event loop: the consumer takes what is queued and otherwise parks on a loop
        event that the result thread sets, so a stream holds no thread of the server's pool between chunks."""
        import asyncio
        with self.lock:
            pr = self.pending.get(request_id)
        if pr is None:
            raise KeyError(request_id)
        loop = asyncio.get_running_loop()
        deadline = time.time() + (timeout_s or self.request_timeout_s)
        ev = asyncio.Event()
        wake = lambda: loop.call_soon_threadsafe(ev.set)   # noqa: E731
        while True:
            try:
                c = pr.chunks.get_nowait()
            except queue.Empty:
                ev.clear()
                pr.wake = wake
                if not pr.chunks.empty():       # a chunk slipped in before the hook was visible
                    pr.wake = None
                    continue
                try:
                    await asyncio.wait_for(ev.wait(), max(0.01, min(1.0, deadline - time.time())))
                except asyncio.TimeoutError:
                    if time.time() > deadline:
                        self.abort_request(request_id)
                        yield ResultChunk("error", b"request timed out", final=True, error_status=500)
                        return
                continue
            if c.modality == "done":
                return
            yield c
            if c.final:
                return

    def collect_results(self, request_id: str, timeout_s: float | None = None) -> dict[str, list[ResultChunk]]:
        out: dict[str, list[ResultChunk]] = {}
        for c in self.iter_result_chunks(request_id, timeout_s):
            out.setdefault(c.modality, []).append(c)
        return out
