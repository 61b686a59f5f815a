"""Media helpers on the host: data-URL / base64 decoding, PCM16 <-> WAV (also open-ended streaming headers),
tensors -> PNG, frames (+audio) -> MP4 through ffmpeg when it is installed.

Reference counterpart: mstar/api_server/media_io.py (272 lines).
"""
from __future__ import annotations

import base64
import io
import shutil
import struct
import subprocess
import tempfile
import wave

import numpy as np
import torch


def decode_media_ref(ref: str, allow_remote: bool = False) -> tuple[bytes, str]:
    """``data:<mime>;base64,<payload>`` or bare base64 -> (bytes, mime). Remote URLs only when allowed."""
    if ref.startswith("data:"):
        head, payload = ref.split(",", 1)
        mime = head[5:].split(";")[0] or "application/octet-stream"
        return base64.b64decode(payload), mime
    if ref.startswith(("http://", "https://")):
        if not allow_remote:
            raise ValueError("remote media references are disabled (MSTAR_ALLOW_REMOTE)")
        import requests
        r = requests.get(ref, timeout=30)
        r.raise_for_status()
        return r.content, r.headers.get("content-type", "application/octet-stream")
    return base64.b64decode(ref), "application/octet-stream"


def ext_for_mime(mime: str) -> str:
    return {"image/png": ".png", "image/jpeg": ".jpg", "image/webp": ".webp", "audio/wav": ".wav", "audio/x-wav": ".wav",
            "audio/mpeg": ".mp3", "video/mp4": ".mp4"}.get(mime, ".bin")


def wav_header(sample_rate: int, channels: int = 1, n_bytes: int | None = None) -> bytes:
    """44-byte PCM16 WAV header. ``n_bytes=None`` writes the open-ended sizes used for streaming."""
    data = 0xFFFFFFFF - 36 if n_bytes is None else n_bytes
    riff = 0xFFFFFFFF if n_bytes is None else 36 + n_bytes
    return (b"RIFF" + struct.pack("<I", riff) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, channels, sample_rate,
            sample_rate * channels * 2, channels * 2, 16) + b"data" + struct.pack("<I", data))


def float_to_pcm16(x: torch.Tensor) -> bytes:
    if x.dtype == torch.int16:          # already quantised by the producer
        if x.device.type != "cpu" or not x.is_contiguous():
            x = x.detach().cpu().contiguous()
        return x.numpy().tobytes()
    return (x.detach().float().clamp(-1, 1) * 32767.0).round().to(torch.int16).cpu().numpy().tobytes()


def pcm16_to_wav(pcm: bytes, sample_rate: int, channels: int = 1) -> bytes:
    return wav_header(sample_rate, channels, len(pcm)) + pcm


def pcm16_to_container(pcm: bytes, sample_rate: int, fmt: str = "wav", channels: int = 1) -> tuple[bytes, str]:
    fmt = (fmt or "wav").lower()
    if fmt == "pcm":
        return pcm, "audio/pcm"
    if fmt == "wav":
        return pcm16_to_wav(pcm, sample_rate, channels), "audio/wav"
    if shutil.which("ffmpeg") is None:
        raise ValueError(f"response_format {fmt!r} needs ffmpeg; use wav or pcm")
    out = subprocess.run(["ffmpeg", "-loglevel", "error", "-f", "s16le", "-ar", str(sample_rate), "-ac", str(channels),
                          "-i", "pipe:0", "-f", fmt, "pipe:1"], input=pcm, capture_output=True, check=True)
    return out.stdout, {"mp3": "audio/mpeg", "flac": "audio/flac", "opus": "audio/opus", "aac": "audio/aac"}.get(fmt, "application/octet-stream")


def read_wav(path_or_bytes) -> tuple[torch.Tensor, int]:
    f = io.BytesIO(path_or_bytes) if isinstance(path_or_bytes, (bytes, bytearray)) else path_or_bytes
    with wave.open(f, "rb") as w:
        sr, ch, n = w.getframerate(), w.getnchannels(), w.getnframes()
        raw = w.readframes(n)
        width = w.getsampwidth()
    if width != 2:
        raise ValueError("only PCM16 WAV input is supported")
    x = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).astype(np.float32) / 32768.0)
    if ch > 1:
        x = x.reshape(-1, ch).mean(-1)
    return x, sr


def tensor_to_png(img: torch.Tensor) -> bytes:
    """[3, H, W] or [H, W, 3]; float in [-1, 1] / [0, 1] or uint8."""
    from PIL import Image
    t = img.detach().cpu()
    if t.dim() == 3 and t.shape[0] in (1, 3):
        t = t.permute(1, 2, 0)
    if t.dtype != torch.uint8:
        t = t.float()
        if t.min() < 0:
            t = (t + 1) / 2
        t = (t.clamp(0, 1) * 255).round().to(torch.uint8)
    arr = t.numpy()
    if arr.shape[-1] == 1:
        arr = arr[..., 0]
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    return buf.getvalue()


def png_to_data_url(png: bytes) -> str:
    return "data:image/png;base64," + base64.b64encode(png).decode()


def frames_to_mp4(frames: torch.Tensor, fps: float = 24.0, audio_pcm: bytes | None = None, sample_rate: int = 24000,
                  channels: int = 1) -> bytes:
    """[T, 3, H, W] frames -> H.264 MP4 (optionally with AAC audio). Needs ffmpeg on the host."""
    if shutil.which("ffmpeg") is None:
        raise RuntimeError("ffmpeg is not installed: cannot encode MP4")
    t = frames.detach().cpu()
    if t.dtype != torch.uint8:
        t = t.float()
        if t.min() < 0:
            t = (t + 1) / 2
        t = (t.clamp(0, 1) * 255).round().to(torch.uint8)
    T, C, H, W = t.shape
    raw = t.permute(0, 2, 3, 1).contiguous().numpy().tobytes()
    with tempfile.TemporaryDirectory() as d:
        cmd = ["ffmpeg", "-loglevel", "error", "-y", "-f", "rawvideo", "-pix_fmt", "rgb24", "-s", f"{W}x{H}", "-r", str(fps),
               "-i", f"{d}/v.raw"]
        open(f"{d}/v.raw", "wb").write(raw)
        if audio_pcm:
            open(f"{d}/a.raw", "wb").write(audio_pcm)
            cmd += ["-f", "s16le", "-ar", str(sample_rate), "-ac", str(channels), "-i", f"{d}/a.raw", "-c:a", "aac", "-shortest"]
        cmd += ["-c:v", "libx264", "-pix_fmt", "yuv420p", f"{d}/out.mp4"]
        subprocess.run(cmd, check=True, capture_output=True)
        return open(f"{d}/out.mp4", "rb").read()


def _to_uint8_frames(frames: torch.Tensor) -> torch.Tensor:
    t = frames.detach().cpu()
    if t.dtype != torch.uint8:
        t = t.float()
        if t.min() < 0:
            t = (t + 1) / 2
        t = (t.clamp(0, 1) * 255).round().to(torch.uint8)
    return t


def frames_to_avi(frames: torch.Tensor, fps: float = 24.0, audio_pcm: bytes | None = None, sample_rate: int = 24000,
                  channels: int = 1, quality: int = 90) -> bytes:
    """[T, 3, H, W] frames -> Motion-JPEG AVI (optionally with one PCM16 audio stream), written here: the
    container needs no external encoder. Audio is interleaved one block per frame."""
    import struct

    from PIL import Image
    t = _to_uint8_frames(frames)
    T, C, H, W = t.shape
    arr = t.permute(0, 2, 3, 1).contiguous().numpy()
    jpgs = []
    for i in range(T):
        buf = io.BytesIO()
        Image.fromarray(arr[i]).save(buf, format="JPEG", quality=quality)
        jpgs.append(buf.getvalue())

    def chunk(cc: bytes, data: bytes) -> bytes:
        return cc + struct.pack("<I", len(data)) + data + (b"\x00" if len(data) & 1 else b"")

    def lst(kind: bytes, data: bytes) -> bytes:
        return b"LIST" + struct.pack("<I", len(data) + 4) + kind + data

    usec = int(round(1e6 / fps))
    n_streams = 2 if audio_pcm else 1
    max_jpg = max(len(j) for j in jpgs)
    avih = struct.pack("<IIIIIIIIIIIIII", usec, int(max_jpg * fps), 0, 0x10, T, 0, n_streams, max_jpg, W, H, 0, 0, 0, 0)
    scale = 1000
    strh_v = struct.pack("<4s4sIHHIIIIIIIIhhhh", b"vids", b"MJPG", 0, 0, 0, 0, scale, int(round(fps * scale)), 0, T,
                         max_jpg, 0xFFFFFFFF, 0, 0, 0, W, H)
    strf_v = struct.pack("<IiiHH4sIiiII", 40, W, H, 1, 24, b"MJPG", W * H * 3, 0, 0, 0, 0)
    hdrl = chunk(b"avih", avih) + lst(b"strl", chunk(b"strh", strh_v) + chunk(b"strf", strf_v))
    blocks = []
    if audio_pcm:
        bps = 2 * channels
        n_samples = len(audio_pcm) // bps
        strh_a = struct.pack("<4s4sIHHIIIIIIIIhhhh", b"auds", b"\x01\x00\x00\x00", 0, 0, 0, 0, 1, sample_rate, 0,
                             n_samples, sample_rate * bps, 0xFFFFFFFF, bps, 0, 0, 0, 0)
        strf_a = struct.pack("<HHIIHH", 1, channels, sample_rate, sample_rate * bps, bps, 16)
        hdrl += lst(b"strl", chunk(b"strh", strh_a) + chunk(b"strf", strf_a))
        per = (n_samples + T - 1) // T * bps
        blocks = [audio_pcm[i * per:(i + 1) * per] for i in range(T)]
    movi, idx, off = b"", b"", 4
    for i, j in enumerate(jpgs):
        c = chunk(b"00dc", j)
        idx += struct.pack("<4sIII", b"00dc", 0x10, off, len(j))
        movi += c
        off += len(c)
        if blocks and blocks[i]:
            c = chunk(b"01wb", blocks[i])
            idx += struct.pack("<4sIII", b"01wb", 0x10, off, len(blocks[i]))
            movi += c
            off += len(c)
    body = b"AVI " + lst(b"hdrl", hdrl) + lst(b"movi", movi) + chunk(b"idx1", idx)
    return b"RIFF" + struct.pack("<I", len(body)) + body


def frames_to_video(frames: torch.Tensor, fps: float = 24.0, audio_pcm: bytes | None = None,
                    sample_rate: int = 24000, channels: int = 1) -> tuple[bytes, str]:
    """(bytes, mime): H.264 MP4 when ffmpeg is on the host, else Motion-JPEG AVI."""
    if shutil.which("ffmpeg") is not None:
        return frames_to_mp4(frames, fps, audio_pcm, sample_rate, channels), "video/mp4"
    return frames_to_avi(frames, fps, audio_pcm, sample_rate, channels), "video/x-msvideo"
