"""Shapes of the Orpheus-3B TTS backbone (Llama-3.2-3B with the audio-token vocabulary).
Reference: mstar/model/orpheus/config.py, mstar/model/orpheus/components/language_model.py."""
import torch

from .decoder import DecoderConfig


def orpheus_3b_config(dtype=torch.bfloat16) -> DecoderConfig:
    return DecoderConfig(hidden_size=3072, num_layers=28, num_heads=24, num_kv_heads=8, head_dim=128,
                         intermediate_size=8192, vocab_size=156940, rms_eps=1e-5, rope_theta=500000.0,
                         rope_llama3=dict(factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=8192),
                         tie_embeddings=True, dtype=dtype)
