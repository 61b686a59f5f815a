"""name -> model class (lazy import), plus the Hugging Face ids the reference serves under these names.
Reference counterpart: mstar/model/registry.py (``MODEL_REGISTRY``, ``HF_MODELS``, ``get_model_class``)."""
from __future__ import annotations

import importlib

MODEL_REGISTRY: dict[str, str] = {
    "tiny": "mstar_b200.models.tiny_model:TinyLM",
    "orpheus": "mstar_b200.models.orpheus:OrpheusModel",
    "bagel": "mstar_b200.models.bagel:BagelModel",
    "qwen3_omni": "mstar_b200.models.qwen3_omni:Qwen3OmniModel",
    "cosmos3": "mstar_b200.models.cosmos3:Cosmos3Model",
    "cosmos3_droid": "mstar_b200.models.cosmos3:Cosmos3DroidModel",
    "cosmos3_super": "mstar_b200.models.cosmos3:Cosmos3SuperModel",
    "wan22": "mstar_b200.models.wan22:Wan22Model",
    "pi05": "mstar_b200.models.pi05:Pi05Model",
    "pi05_droid": "mstar_b200.models.pi05:Pi05DroidModel",
    "vjepa2": "mstar_b200.models.vjepa2:VJepa2Model",
    "vjepa2_ac": "mstar_b200.models.vjepa2:VJepa2ACModel",
    "qwen3_tts": "mstar_b200.models.qwen3_tts:Qwen3TTSModel",
    "whisper_large": "mstar_b200.models.whisper:WhisperModel",
    "higgs_audio": "mstar_b200.models.higgs_audio:HiggsAudioModel",
}

HF_MODELS: dict[str, str] = {
    "orpheus": "canopylabs/orpheus-3b-0.1-ft",
    "bagel": "ByteDance-Seed/BAGEL-7B-MoT",
    "qwen3_omni": "Qwen/Qwen3-Omni-30B-A3B-Instruct",
    "cosmos3": "nvidia/Cosmos-3-Nano",
    "wan22": "Wan-AI/Wan2.2-TI2V-5B-Diffusers",
    "pi05": "lerobot/pi05_base",
    "vjepa2": "facebook/vjepa2-vitl-fpc64-256",
    "qwen3_tts": "Qwen/Qwen3-TTS",
    "whisper_large": "openai/whisper-large-v3",
    "higgs_audio": "bosonai/higgs-audio-v3-stt",
}


def get_model_class(name: str):
    if name not in MODEL_REGISTRY:
        raise KeyError(f"unknown model {name!r}; known: {sorted(MODEL_REGISTRY)}")
    mod, cls = MODEL_REGISTRY[name].split(":")
    return getattr(importlib.import_module(mod), cls)
