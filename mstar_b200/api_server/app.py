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


def create_app(server: APIServer, allow_remote_media: bool = False) -> FastAPI:
    app = FastAPI(title="mstar-b200")
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
            if m not in ("text", "audio", "image", "video", "action", "embedding"):
                raise HTTPException(400, f"unknown modality {m!r}")
        rid = server.submit_request(text, blobs, in_mods, out_mods, kw, request_id)
        if streaming:
            def gen():
                for c in server.iter_result_chunks(rid):
                    d = {"modality": c.modality, "data": base64.b64encode(c.data).decode(), "metadata": c.metadata}
                    if c.error_status:
                        d["error_status"] = c.error_status
                    yield json.dumps(d) + "\n"
            return StreamingResponse(gen(), media_type="application/x-ndjson")
        res = _collect(rid)
        return {"request_id": rid, "outputs": {m: [{"data": base64.b64encode(c.data).decode(), "metadata": c.metadata}
                                                   for c in cs] for m, cs in res.items()}}

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
            def sse():
                first = True
                for c in server.iter_result_chunks(rid):
                    if c.modality == "error":
                        yield f"data: {json.dumps({'error': {'message': c.data.decode(errors='replace'), 'code': c.error_status}})}\n\n"
                        break
                    delta = {"role": "assistant"} if first else {}
                    first = False
                    if c.modality == "text":
                        delta["content"] = c.data.decode(errors="replace")
                    elif c.modality == "audio":
                        delta["audio"] = {"id": cid, "data": base64.b64encode(c.data).decode()}
                    elif c.modality == "image":
                        delta["content"] = [{"type": "image_url", "image_url": {"url": png_to_data_url(c.data)}}]
                    yield "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                                 "model": model_name, "choices": [{"index": 0, "delta": delta,
                                                                                   "finish_reason": None}]}) + "\n\n"
                yield "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                             "model": model_name, "choices": [{"index": 0, "delta": {},
                                                                               "finish_reason": "stop"}]}) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
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

            def stream():
                if req.response_format == "wav":
                    yield wav_header(sr, ch, None)
                for c in server.iter_result_chunks(rid):
                    if c.modality == "audio":
                        yield c.data
            return StreamingResponse(stream(), media_type="audio/wav" if req.response_format == "wav" else "audio/pcm")
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
