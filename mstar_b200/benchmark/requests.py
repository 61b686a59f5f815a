"""Request types of the benchmark client and their synthetic inputs. Every type maps to one call of the native
``POST /generate`` endpoint (multipart form, NDJSON stream).

Reference counterparts: request types and dataset adapters (benchmark/base.py, benchmark/dataset.py); datasets that
need downloads are replaced by synthetic inputs of the same shape.
"""
from __future__ import annotations

import io
import json
import random
import struct
import wave
from dataclasses import dataclass, field

REQUEST_TYPES = {
    # name: (input modalities besides text, output modalities)
    "t2t": ([], ["text"]),             # text -> text
    "i2t": (["image"], ["text"]),      # image + text -> text
    "a2t": (["audio"], ["text"]),      # audio + text -> text (ASR / audio understanding)
    "tts": ([], ["audio"]),            # text -> speech
    "t2s": ([], ["text", "audio"]),    # text -> text + speech (omni models)
    "t2i": ([], ["image"]),            # text -> image
    "i2i": (["image"], ["image"]),     # image edit
    "t2v": ([], ["video"]),            # text -> video
}

_WORDS = ("the quick brown fox jumps over a lazy dog while seven wizards quietly box and judge my vow of "
          "silence under bright northern lights").split()


@dataclass
class RequestInput:
    request_type: str
    text: str
    files: list = field(default_factory=list)          # (filename, bytes)
    output_modalities: list = field(default_factory=lambda: ["text"])
    model_kwargs: dict = field(default_factory=dict)

    def form(self):
        data = {"text": self.text, "output_modalities": ",".join(self.output_modalities), "streaming": "true",
                "model_kwargs": json.dumps(self.model_kwargs)}
        return data, list(self.files)


def synthetic_png(width: int, height: int, rng: random.Random) -> bytes:
    """A valid PNG of uniform noise without any imaging library (stored deflate blocks)."""
    import zlib
    raw = bytearray()
    for _ in range(height):
        raw.append(0)
        raw.extend(rng.getrandbits(8) for _ in range(width * 3))

    def chunk(tag, data):
        c = struct.pack(">I", len(data)) + tag + data
        return c + struct.pack(">I", zlib.crc32(tag + data) & 0xffffffff)
    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", width, height, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(bytes(raw), 1)) + chunk(b"IEND", b""))


def synthetic_wav(seconds: float, rng: random.Random, sample_rate: int = 16000) -> bytes:
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sample_rate)
        w.writeframes(b"".join(struct.pack("<h", max(-32768, min(32767, int(rng.gauss(0, 3000)))))
                               for _ in range(int(seconds * sample_rate))))
    return buf.getvalue()


def make_requests(request_type: str, n: int, *, seed: int = 0, prompt_words: tuple = (8, 32), max_tokens: int = 128,
                  image_size: int = 448, audio_seconds: float = 5.0, extra_kwargs: dict | None = None,
                  numeric_prompts: bool = False) -> list[RequestInput]:
    """``numeric_prompts`` writes prompts as space-separated token ids (for servers started without a tokenizer)."""
    if request_type not in REQUEST_TYPES:
        raise ValueError(f"unknown request type {request_type!r}; one of {sorted(REQUEST_TYPES)}")
    ins, outs = REQUEST_TYPES[request_type]
    rng = random.Random(seed)
    reqs = []
    for i in range(n):
        k = rng.randint(*prompt_words)
        text = (" ".join(str(rng.randrange(1000, 30000)) for _ in range(k)) if numeric_prompts
                else " ".join(rng.choice(_WORDS) for _ in range(k)))
        files = []
        if "image" in ins:
            files.append((f"in{i}.png", synthetic_png(image_size, image_size, rng)))
        if "audio" in ins:
            files.append((f"in{i}.wav", synthetic_wav(audio_seconds, rng)))
        kw = {"max_tokens": max_tokens, **(extra_kwargs or {})}
        reqs.append(RequestInput(request_type, text, files, list(outs), kw))
    return reqs
