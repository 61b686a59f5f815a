"""Python SDK over the native ``/generate`` endpoint (plus sugar for chat, images and speech).
Reference counterpart: ``MStarClient`` (mstar/client/client.py:43-158)."""
from __future__ import annotations

import base64
import json
import os

import requests

from .types import AudioBuffer, AudioChunk, GenerateResult, ImageChunk, TextChunk, VideoChunk


class MStarClient:
    def __init__(self, base_url: str = "http://127.0.0.1:8000", timeout: float = 600.0, session=None):
        self.base_url, self.timeout = base_url.rstrip("/"), timeout
        self.session = session or requests.Session()

    def health(self) -> dict:
        r = self.session.get(self.base_url + "/health", timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    @staticmethod
    def _files(images, audio, video):
        out = []
        for group in (images, audio, video):
            for item in group or []:
                if isinstance(item, (bytes, bytearray)):
                    out.append(("files", ("upload.bin", bytes(item))))
                elif isinstance(item, tuple):
                    out.append(("files", item))
                else:
                    out.append(("files", (os.path.basename(item), open(item, "rb").read())))
        return out

    def _post(self, text, images, audio, video, output_modalities, input_modalities, stream, request_id, model_kwargs):
        data = {"output_modalities": ",".join(output_modalities or ["text"]), "streaming": "true" if stream else "false",
                "model_kwargs": json.dumps(model_kwargs or {})}
        if text is not None:
            data["text"] = text
        if input_modalities:
            data["input_modalities"] = ",".join(input_modalities)
        if request_id:
            data["request_id"] = request_id
        files = self._files(images, audio, video) or None
        return self.session.post(self.base_url + "/generate", data=data, files=files, stream=stream, timeout=self.timeout)

    @staticmethod
    def _chunk(d: dict):
        blob = base64.b64decode(d.get("data", ""))
        m, md = d.get("modality"), d.get("metadata", {})
        if m == "text":
            return TextChunk(blob.decode(errors="replace"), md)
        if m == "image":
            return ImageChunk(blob, md)
        if m == "audio":
            return AudioChunk(blob, md)
        if m == "video":
            return VideoChunk(blob, md)
        if m == "error":
            raise RuntimeError(f"request failed ({d.get('error_status')}): {blob.decode(errors='replace')}")
        return None

    def stream(self, text=None, images=None, audio=None, video=None, output_modalities=None, input_modalities=None,
               request_id=None, **model_kwargs):
        r = self._post(text, images, audio, video, output_modalities, input_modalities, True, request_id, model_kwargs)
        r.raise_for_status()
        for line in r.iter_lines():
            if line:
                c = self._chunk(json.loads(line))
                if c is not None:
                    yield c

    def generate(self, text=None, images=None, audio=None, video=None, output_modalities=None, input_modalities=None,
                 stream=False, request_id=None, **model_kwargs):
        if stream:
            return self.stream(text, images, audio, video, output_modalities, input_modalities, request_id, **model_kwargs)
        r = self._post(text, images, audio, video, output_modalities, input_modalities, False, request_id, model_kwargs)
        if r.status_code >= 400:
            raise RuntimeError(f"request failed ({r.status_code}): {r.text}")
        doc = r.json()
        res = GenerateResult(request_id=doc.get("request_id", ""), raw=doc)
        outs = doc.get("outputs", {})
        res.text = "".join(base64.b64decode(c["data"]).decode(errors="replace") for c in outs.get("text", []))
        res.images = [base64.b64decode(c["data"]) for c in outs.get("image", [])]
        res.videos = [base64.b64decode(c["data"]) for c in outs.get("video", [])]
        res.audio = AudioBuffer(b"".join(base64.b64decode(c["data"]) for c in outs.get("audio", [])))
        return res

    def chat(self, text: str, **kw) -> str:
        return self.generate(text, **kw).text

    def generate_image(self, prompt: str, **kw) -> bytes:
        return self.generate(prompt, output_modalities=["image"], **kw).images[0]

    def tts(self, text: str, **kw) -> AudioBuffer:
        return self.generate(text, output_modalities=["audio"], **kw).audio
