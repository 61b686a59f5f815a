"""HTTP surface (FastAPI): native ``POST /generate`` (multipart form; NDJSON stream or one JSON document),
``GET /health``, ``GET /metrics`` (Prometheus text), and the OpenAI-compatible routes ``/v1/models``,
``/v1/chat/completions`` (SSE), ``/v1/audio/speech`` (streaming WAV), ``/v1/images/generations``,
``/v1/images/edits``, ``/v1/videos/generations``.

Reference counterparts: mstar/api_server/entrypoint.py:680-817 (app, /generate, /health), openai/router.py:76-135
and serving_chat / serving_images / serving_speech / serving_videos. ``/metrics`` is an addition.
"""
from __future__ import annotations

import base64
import json
import time
import uuid

from fastapi import FastAPI, File, Form, HTTPException, Request, UploadFile
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

from .media_io import pcm16_to_container, pcm16_to_wav, png_to_data_url, wav_header
from .openai.adapters import get_adapter
from .openai.protocol import (ChatCompletionRequest, ImageGenerationRequest, ModelCard, ModelList, SpeechRequest,
                              VideoGenerationRequest)
from .server import APIServer


DIRECT_STREAM_EXT = "mstar.direct_stream"


class ChunkStream(Response):
    """Streaming reply built from a request's result chunks. ``fmt(chunk)`` returns the pieces (bytes) a chunk turns
    into and whether the stream ends with it; ``head`` / ``tail`` frame the stream.

    Under a transport that offers the ``mstar.direct_stream`` ASGI extension (the C++ frontend's bridge) the pieces
    are handed to the transport on the thread that received them from the workers: between the reply's start and
    its end the event loop does nothing for this stream. Any other ASGI server gets an ordinary async body iterator.
    ``raw(chunk)`` -> (prefix, data, suffix) or None, when given, states a chunk as prefix + base64(data) + suffix: a
    transport whose sink has a ``b64`` method then encodes the binary field itself and may send the chunks of many
    requests as one frame.
    """

    def __init__(self, server: APIServer, rid: str, fmt, media_type: str, head=(), tail=(), raw=None):
        super().__init__(content=None, media_type=media_type)
        self.raw_headers = [h for h in self.raw_headers if h[0] != b"content-length"]
        self.server, self.rid, self.fmt, self.head, self.tail = server, rid, fmt, list(head), tail
        self.raw = raw

    async def _body(self):
        for piece in self.head:
            yield piece
        async for c in self.server.aiter_result_chunks(self.rid):
            pieces, last = self.fmt(c)
            for piece in pieces:
                yield piece
            if last:
                break
        for piece in (self.tail() if callable(self.tail) else self.tail):
            yield piece

    async def __call__(self, scope, receive, send):
        direct = (scope.get("extensions") or {}).get(DIRECT_STREAM_EXT)
        if direct is None:
            resp = StreamingResponse(self._body(), media_type=self.media_type)
            await resp(scope, receive, send)
            return
        import asyncio
        loop, done = asyncio.get_running_loop(), asyncio.Event()
        await send({"type": "http.response.start", "status": 200, "headers": self.raw_headers})
        for piece in self.head:
            direct(piece)
        state = {"open": True}

        b64 = getattr(direct, "b64", None) if self.raw is not None else None

        def sink(c):                    # runs on the server's result thread
            if not state["open"]:
                return
            last = True
            if c.modality != "done":
                parts = self.raw(c) if b64 is not None else None
                if parts is not None:   # the transport encodes the binary field and sends a batch's chunks together
                    b64(*parts)
                    last = False
                else:
                    pieces, last = self.fmt(c)
                    for piece in pieces:
                        direct(piece)
                last = last or c.final
            if last:
                state["open"] = False
                for piece in (self.tail() if callable(self.tail) else self.tail):
                    direct(piece)
                loop.call_soon_threadsafe(done.set)
        self.server.attach_sink(self.rid, sink)
        getattr(direct, "flush", lambda: None)()      # chunks that were queued before the sink took over
        try:
            await done.wait()
        except asyncio.CancelledError:  # the client went away: stop generating for it
            state["open"] = False
            self.server.abort_request(self.rid)
            raise
        finally:
            self.server.detach_sink(self.rid)
        await send({"type": "http.response.body", "body": b"", "more_body": False})


_FORM_FIELDS = {"text", "input_modalities", "output_modalities", "streaming", "model_kwargs", "request_id"}


def _simple_form(body: bytes, content_type: str) -> dict[str, str] | None:
    """The fields of a form body that holds plain text fields only (``application/x-www-form-urlencoded``, or
    ``multipart/form-data`` without file parts); None when it holds anything else (a file part, an unknown or repeated
    field, another encoding) or is not well formed."""
    ct = (content_type or "").lower()
    if ct.startswith("application/x-www-form-urlencoded"):
        from urllib.parse import parse_qsl
        try:
            pairs = parse_qsl(body.decode("utf-8"), keep_blank_values=True, strict_parsing=bool(body))
        except (UnicodeDecodeError, ValueError):
            return None
        out_: dict[str, str] = {}
        for k, v in pairs:
            if k not in _FORM_FIELDS or k in out_:
                return None
            out_[k] = v
        return out_
    if not ct.startswith("multipart/form-data"):
        return None
    b = None
    for item in content_type.split(";")[1:]:
        k, _, v = item.strip().partition("=")
        if k.lower() == "boundary":
            b = v.strip().strip('"')
    if not b:
        return None
    delim = b"--" + b.encode()
    parts = body.split(delim)
    if len(parts) < 3 or not parts[-1].lstrip().startswith(b"--"):
        return None
    out: dict[str, str] = {}
    for part in parts[1:-1]:
        head, sep, value = part.partition(b"\r\n\r\n")
        if not sep or not head.startswith(b"\r\n") or not value.endswith(b"\r\n"):
            return None
        name = None
        for line in head.strip().split(b"\r\n"):
            key, _, rest = line.partition(b":")
            if key.strip().lower() == b"content-disposition":
                if b"filename" in rest:
                    return None
                for item in rest.split(b";")[1:]:
                    k, _, v = item.strip().partition(b"=")
                    if k == b"name":
                        name = v.strip().strip(b'"').decode("utf-8", "replace")
            elif key.strip().lower() == b"content-type" and not rest.strip().lower().startswith(b"text/plain"):
                return None
        if name not in _FORM_FIELDS or name in out:
            return None
        try:
            out[name] = value[:-2].decode("utf-8")
        except UnicodeDecodeError:
            return None
    return out


def create_app(server: APIServer, allow_remote_media: bool = False) -> FastAPI:
    app = FastAPI(title="mstar-b200")
    app.state.mstar_server = server
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    model_name = server.deployment.cfg["model"]
    adapter = get_adapter(model_name)

    def _ready():
        if not server.ready.is_set():
            raise HTTPException(503, "server is starting")

    def _submit(args, request_id=None):
        return server.submit_request(args.text, args.files, args.input_modalities, args.output_modalities,
                                     args.model_kwargs, request_id)

    def _collect(rid):
        res = server.collect_results(rid)
        if "error" in res:
            c = res["error"][0]
            raise HTTPException(c.error_status or 500, c.data.decode(errors="replace"))
        return res

    # ------------------------------------------------------------------ native
    @app.get("/health")
    def health():
        return {"status": "healthy" if server.ready.is_set() else "starting"}

    @app.get("/metrics")
    def metrics():
        lines = []
        for k, v in server.stats.items():
            lines.append(f"mstar_api_requests_{k}_total {v}")
        lines.append(f"mstar_api_pending_requests {sum(1 for p in server.pending.values() if not p.done)}")
        cond = server.deployment.conductor
        if cond is not None:
            lines.append(f"mstar_conductor_running_requests {len(cond.requests)}")
            lines.append(f"mstar_conductor_waiting_requests {len(cond.waiting)}")
        for w in server.deployment.workers:
            for eng in w.engines.engines:
                if hasattr(eng, "cache"):
                    a = eng.cache.alloc
                    lines.append(f'mstar_kv_pages_used{{worker="{w.worker_id}"}} {a.total_pages - a.num_free_pages}')
                    lines.append(f'mstar_kv_pages_total{{worker="{w.worker_id}"}} {a.total_pages}')
                    lines.append(f'mstar_cuda_graph_replays_total{{worker="{w.worker_id}"}} {eng.graph_hits}')
            lines.append(f'mstar_worker_loop_iterations_total{{worker="{w.worker_id}"}} {w.iterations}')
            lines.append(f'mstar_tensor_tx_bytes_total{{worker="{w.worker_id}"}} {w.tensors.tx_bytes}')
        return PlainTextResponse("\n".join(lines) + "\n")

    _MODALITIES = ("text", "audio", "image", "video", "action", "embedding")

    def _generate_stream(rid: str) -> ChunkStream:
        def raw(c):
            # a line is prefix + base64(data) + suffix; base64 needs no JSON escaping, so the line is assembled
            # from bytes instead of serialising a 5 KB string
            tail = b'","metadata":' + json.dumps(c.metadata).encode()
            if c.error_status:
                tail += b',"error_status":' + json.dumps(c.error_status).encode()
            data = c.data if isinstance(c.data, (bytes, bytearray)) else bytes(c.data)
            return b'{"modality":' + json.dumps(c.modality).encode() + b',"data":"', data, tail + b"}\n"

        def fmt(c):
            prefix, data, suffix = raw(c)
            return [prefix + base64.b64encode(data) + suffix], False
        return ChunkStream(server, rid, fmt, "application/x-ndjson", raw=raw)

    @app.post("/generate")
    async def generate(text: str | None = Form(None), files: list[UploadFile] = File(default=[]),
                       input_modalities: str | None = Form(None), output_modalities: str = Form("text"),
                       streaming: bool = Form(True), model_kwargs: str = Form("{}"), request_id: str | None = Form(None)):
        _ready()
        try:
            kw = json.loads(model_kwargs or "{}")
        except json.JSONDecodeError as e:
            raise HTTPException(400, f"model_kwargs is not JSON: {e}") from e
        blobs = []
        for f in files:
            name = (f.filename or "upload").replace("\\", "/").split("/")[-1]
            blobs.append((f"{uuid.uuid4().hex}_{name}", await f.read()))
        in_mods = [m.strip() for m in input_modalities.split(",")] if input_modalities else None
        out_mods = [m.strip() for m in output_modalities.split(",") if m.strip()]
        for m in out_mods + (in_mods or []):
            if m not in _MODALITIES:
                raise HTTPException(400, f"unknown modality {m!r}")
        rid = server.submit_request(text, blobs, in_mods, out_mods, kw, request_id)
        if streaming:
            return _generate_stream(rid)
        res = _collect(rid)
        return {"request_id": rid, "outputs": {m: [{"data": base64.b64encode(c.data).decode(), "metadata": c.metadata}
                                                   for c in cs] for m, cs in res.items()}}

    def fast_generate(body: bytes, content_type: str):
        """The common streaming ``POST /generate`` (text fields only, no uploads) without the framework's form parsing,
        validation layers and routing: returns the streaming response, or None for anything that needs the full route
        (uploads, non-streaming replies, malformed input — the route then produces the proper error). A transport
        that has the whole body in hand (the C++ frontend's bridge) may try this first; 0.35 instead of 1.0 ms per
        request, which is what first-audio latency pays per queued request when hundreds arrive together."""
        if not server.ready.is_set():
            return None
        fields = _simple_form(body, content_type)
        if fields is None or fields.get("streaming", "true").lower() not in ("true", "1", "yes", "on"):
            return None
        try:
            kw = json.loads(fields.get("model_kwargs") or "{}")
        except json.JSONDecodeError:
            return None
        in_mods = [m.strip() for m in fields["input_modalities"].split(",")] if fields.get("input_modalities") else None
        out_mods = [m.strip() for m in fields.get("output_modalities", "text").split(",") if m.strip()]
        if any(m not in _MODALITIES for m in out_mods + (in_mods or [])) or not isinstance(kw, dict):
            return None
        return _generate_stream(server.submit_request(fields.get("text"), [], in_mods, out_mods, kw, fields.get("request_id")))

    app.state.fast_routes = {("POST", "/generate"): fast_generate}

    # ------------------------------------------------------------------ OpenAI-compatible
    @app.get("/v1/models")
    def models():
        return ModelList(data=[ModelCard(id=model_name, created=int(time.time()))])

    @app.post("/v1/chat/completions")
    def chat(req: ChatCompletionRequest, http: Request):
        _ready()
        args = adapter.chat(req, allow_remote_media)
        rid = _submit(args)
        cid, created = "chatcmpl-" + rid[:24], int(time.time())
        sr = server.model.get_output_sample_rate()
        if req.stream:
            st = {"first": True}

            def fmt(c):
                if c.modality == "error":
                    return [f"data: {json.dumps({'error': {'message': c.data.decode(errors='replace'), 'code': c.error_status}})}\n\n".encode()], True
                delta = {"role": "assistant"} if st["first"] else {}
                st["first"] = False
                if c.modality == "text":
                    delta["content"] = c.data.decode(errors="replace")
                elif c.modality == "audio":
                    delta["audio"] = {"id": cid, "data": base64.b64encode(c.data).decode()}
                elif c.modality == "image":
                    delta["content"] = [{"type": "image_url", "image_url": {"url": png_to_data_url(c.data)}}]
                return [("data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                                "model": model_name, "choices": [{"index": 0, "delta": delta,
                                                                                  "finish_reason": None}]}) + "\n\n").encode()], False
            tail = [("data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                            "model": model_name, "choices": [{"index": 0, "delta": {},
                                                                              "finish_reason": "stop"}]}) + "\n\n").encode(),
                    b"data: [DONE]\n\n"]
            return ChunkStream(server, rid, fmt, "text/event-stream", tail=tail)
        res = _collect(rid)
        msg: dict = {"role": "assistant", "content": b"".join(c.data for c in res.get("text", [])).decode(errors="replace")}
        if "audio" in res:
            pcm = b"".join(c.data for c in res["audio"])
            msg["audio"] = {"id": cid, "data": base64.b64encode(pcm16_to_wav(pcm, sr)).decode(), "transcript": msg["content"]}
        if "image" in res:
            msg["content"] = ([{"type": "text", "text": msg["content"]}] if msg["content"] else []) + \
                [{"type": "image_url", "image_url": {"url": png_to_data_url(c.data)}} for c in res["image"]]
        return {"id": cid, "object": "chat.completion", "created": created, "model": model_name,
                "choices": [{"index": 0, "message": msg, "finish_reason": "stop"}],
                "usage": {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}}

    @app.post("/v1/audio/speech")
    def speech(req: SpeechRequest):
        _ready()
        rid = _submit(adapter.speech(req))
        sr, ch = server.model.get_output_sample_rate(), server.model.get_output_audio_channels()
        if req.stream:
            if req.response_format not in ("wav", "pcm"):
                raise HTTPException(422, "streaming supports wav and pcm only")

            def fmt(c):
                return ([bytes(c.data)] if c.modality == "audio" and c.data else []), False
            return ChunkStream(server, rid, fmt, "audio/wav" if req.response_format == "wav" else "audio/pcm",
                               head=[wav_header(sr, ch, None)] if req.response_format == "wav" else [])
        res = _collect(rid)
        pcm = b"".join(c.data for c in res.get("audio", []))
        try:
            blob, mime = pcm16_to_container(pcm, sr, req.response_format, ch)
        except ValueError as e:
            raise HTTPException(422, str(e)) from e
        return Response(blob, media_type=mime)

    @app.post("/v1/images/generations")
    def images(req: ImageGenerationRequest):
        _ready()
        rids = [_submit(adapter.image(req, i)) for i in range(max(1, req.n or 1))]
        data = []
        for rid in rids:
            for c in _collect(rid).get("image", []):
                data.append({"b64_json": base64.b64encode(c.data).decode()})
        return {"created": int(time.time()), "data": data}

    @app.post("/v1/images/edits")
    async def image_edits(prompt: str = Form(...), image: list[UploadFile] = File(...), n: int = Form(1),
                          size: str | None = Form(None), seed: int | None = Form(None)):
        _ready()
        files = [(f"{uuid.uuid4().hex}_{(f.filename or 'image.png').split('/')[-1]}", await f.read()) for f in image]
        data = []
        for i in range(max(1, n)):
            kw = {}
            if size:
                w, h = size.lower().split("x")
                kw.update(width=int(w), height=int(h))
            if seed is not None:
                kw["seed"] = seed + i
            rid = server.submit_request(prompt, files, None, ["image"], kw)
            for c in _collect(rid).get("image", []):
                data.append({"b64_json": base64.b64encode(c.data).decode()})
        return {"created": int(time.time()), "data": data}

    @app.post("/v1/videos/generations")
    def videos(req: VideoGenerationRequest):
        _ready()
        rids = [_submit(adapter.video(req, i, allow_remote_media)) for i in range(max(1, req.n or 1))]
        data = []
        for rid in rids:
            res = _collect(rid)
            for c in res.get("video", []):
                data.append({"b64_json": base64.b64encode(c.data).decode()})
        return {"created": int(time.time()), "data": data}

    @app.exception_handler(HTTPException)
    async def http_exc(_: Request, exc: HTTPException):
        return JSONResponse({"error": {"message": exc.detail, "code": exc.status_code}}, status_code=exc.status_code)

    return app
