"""Result types of the Python SDK. Reference counterpart: mstar/client/types.py."""
from __future__ import annotations

import io
import struct
import wave
from dataclasses import dataclass, field


@dataclass
class TextChunk:
    text: str
    metadata: dict = field(default_factory=dict)


@dataclass
class ImageChunk:
    png: bytes
    metadata: dict = field(default_factory=dict)


@dataclass
class AudioChunk:
    pcm16: bytes
    metadata: dict = field(default_factory=dict)


@dataclass
class VideoChunk:
    mp4: bytes
    metadata: dict = field(default_factory=dict)


@dataclass
class AudioBuffer:
    pcm16: bytes = b""
    sample_rate: int = 24000
    channels: int = 1

    def wav_bytes(self) -> bytes:
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(self.channels)
            w.setsampwidth(2)
            w.setframerate(self.sample_rate)
            w.writeframes(self.pcm16)
        return buf.getvalue()

    def to_wav(self, path: str) -> str:
        with open(path, "wb") as f:
            f.write(self.wav_bytes())
        return path

    def to_numpy(self):
        import numpy as np
        return np.frombuffer(self.pcm16, dtype=np.int16).astype(np.float32) / 32768.0

    @property
    def duration_s(self) -> float:
        return len(self.pcm16) / 2 / self.channels / self.sample_rate


@dataclass
class GenerateResult:
    request_id: str = ""
    text: str = ""
    images: list[bytes] = field(default_factory=list)
    audio: AudioBuffer = field(default_factory=AudioBuffer)
    videos: list[bytes] = field(default_factory=list)
    raw: dict = field(default_factory=dict)

    def save_image(self, path: str, index: int = 0) -> str:
        with open(path, "wb") as f:
            f.write(self.images[index])
        return path

    def save_audio(self, path: str) -> str:
        return self.audio.to_wav(path)
