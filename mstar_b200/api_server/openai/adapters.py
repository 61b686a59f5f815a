"""Per-model translation of OpenAI request fields into ``SubmitArgs`` (prompt text, media files, modalities,
model_kwargs). Reference counterparts: ``flatten_messages`` (mstar/api_server/openai/adapters.py:51-109),
``_apply_sampling`` (:119-154), ``ADAPTER_REGISTRY`` (:433-441)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..media_io import decode_media_ref, ext_for_mime


@dataclass
class SubmitArgs:
    text: str | None = None
    files: list[tuple[str, bytes]] = field(default_factory=list)
    input_modalities: list[str] | None = None
    output_modalities: list[str] = field(default_factory=lambda: ["text"])
    model_kwargs: dict = field(default_factory=dict)


def flatten_messages(messages: list, allow_remote: bool = False) -> tuple[str, list[tuple[str, bytes]]]:
    """Chat messages -> one prompt string (role-tagged turns) and the media parts in order of appearance."""
    lines, files = [], []
    for m in messages:
        role = m.role if hasattr(m, "role") else m["role"]
        content = m.content if hasattr(m, "content") else m.get("content")
        if isinstance(content, str) or content is None:
            text = content or ""
        else:
            parts = []
            for part in content:
                kind = part.get("type")
                if kind == "text":
                    parts.append(part.get("text", ""))
                elif kind in ("image_url", "audio_url", "video_url", "input_audio"):
                    ref = part.get(kind, {})
                    url = ref.get("url") if isinstance(ref, dict) else ref
                    if kind == "input_audio":
                        url = "data:audio/wav;base64," + ref.get("data", "")
                    blob, mime = decode_media_ref(url, allow_remote)
                    ext = ext_for_mime(mime)
                    if ext == ".bin":
                        ext = {"image_url": ".png", "audio_url": ".wav", "input_audio": ".wav", "video_url": ".mp4"}[kind]
                    files.append((f"part{len(files)}{ext}", blob))
            text = "\n".join(p for p in parts if p)
        lines.append(f"{role}: {text}" if role != "user" or len(messages) > 1 else text)
    return "\n".join(lines), files


def _apply_sampling(req, kw: dict) -> None:
    for src, dst in (("temperature", "temperature"), ("top_p", "top_p"), ("seed", "seed")):
        v = getattr(req, src, None)
        if v is not None:
            kw[dst] = v
    mt = getattr(req, "max_completion_tokens", None) or getattr(req, "max_tokens", None)
    if mt is not None:
        kw["max_tokens"] = int(mt)
    extra = getattr(req, "model_extra", None) or {}
    for k, v in extra.items():
        kw.setdefault(k, v)


def _size(req, kw: dict) -> None:
    s = getattr(req, "size", None)
    if s:
        w, h = s.lower().split("x")
        kw["width"], kw["height"] = int(w), int(h)


class Adapter:
    """Default adapter: text chat in, text out."""
    chat_output_modalities = ["text"]

    def chat(self, req, allow_remote=False) -> SubmitArgs:
        text, files = flatten_messages(req.messages, allow_remote)
        kw: dict = {}
        _apply_sampling(req, kw)
        mods = list(req.modalities or self.chat_output_modalities)
        if req.audio and req.audio.get("voice"):
            kw["voice"] = req.audio["voice"]
        return SubmitArgs(text, files, None, mods, kw)

    def speech(self, req) -> SubmitArgs:
        kw: dict = {}
        _apply_sampling(req, kw)
        if req.voice:
            kw["voice"] = req.voice
        return SubmitArgs(req.input, [], ["text"], ["audio"], kw)

    def image(self, req, index: int = 0) -> SubmitArgs:
        kw: dict = {}
        _apply_sampling(req, kw)
        _size(req, kw)
        if req.seed is not None:
            kw["seed"] = int(req.seed) + index
        return SubmitArgs(req.prompt, [], ["text"], ["image"], kw)

    def video(self, req, index: int = 0, allow_remote=False) -> SubmitArgs:
        kw: dict = {}
        _apply_sampling(req, kw)
        _size(req, kw)
        if req.num_frames:
            kw["num_frames"] = int(req.num_frames)
        if req.fps:
            kw["fps"] = float(req.fps)
        if req.seed is not None:
            kw["seed"] = int(req.seed) + index
        files = []
        for ref, ext in ((req.image, ".png"), (req.video, ".mp4")):
            if ref:
                blob, mime = decode_media_ref(ref, allow_remote)
                files.append((f"cond{len(files)}{ext if ext_for_mime(mime) == '.bin' else ext_for_mime(mime)}", blob))
        return SubmitArgs(req.prompt, files, None, ["video"], kw)


class OrpheusAdapter(Adapter):
    chat_output_modalities = ["audio"]


class Qwen3OmniAdapter(Adapter):
    chat_output_modalities = ["text"]


class BagelAdapter(Adapter):
    pass


class Cosmos3Adapter(Adapter):
    chat_output_modalities = ["image"]


class Wan22Adapter(Adapter):
    chat_output_modalities = ["video"]


ADAPTER_REGISTRY: dict[str, type[Adapter]] = {
    "orpheus": OrpheusAdapter, "qwen3_omni": Qwen3OmniAdapter, "bagel": BagelAdapter, "cosmos3": Cosmos3Adapter,
    "cosmos3_droid": Cosmos3Adapter, "cosmos3_super": Cosmos3Adapter, "wan22": Wan22Adapter, "qwen3_tts": OrpheusAdapter,
}


def get_adapter(model_name: str) -> Adapter:
    return ADAPTER_REGISTRY.get(model_name, Adapter)()
