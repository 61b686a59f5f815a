"""Higgs-Audio v3 class speech-to-text: a Whisper-style audio encoder over fixed 4-second chunks whose frames are
projected to the width of a Qwen3-1.7B class decoder and spliced into the prompt at audio placeholder tokens.

Walks: ``prefill_text`` (no audio), ``prefill_audio`` (encoder, then one packed prefill), ``decode``.
Reference counterparts: mstar/model/higgs_audio/higgs_audio_model.py (519 lines), submodules.py (218).
"""
from __future__ import annotations

import torch

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import GraphEdge, GraphNode
from .base import small_scale, EngineType, Model
from .decoder import DecoderConfig, DecoderLM
from .encoders import AudioEncoder, EncoderConfig, log_mel_spectrogram
from .llm_common import LMStateMachine, MultimodalDecoderSubmodule, expand_placeholders, lm_walks
from .submodule_base import NodeSubmodule

AUDIO_TOKEN, AUDIO_BOS, AUDIO_EOS, EOS = 151665, 151666, 151667, 151645
CHUNK_S = 4.0


class ChunkedAudioEncoderSubmodule(NodeSubmodule):
    """Splits the waveform into fixed chunks (the last one zero-padded) and encodes them as one packed batch."""

    def __init__(self, enc: AudioEncoder, device, n_mels: int, chunk_s: float = CHUNK_S):
        super().__init__(device, enc.c.dtype)
        self.enc, self.n_mels, self.chunk = enc, n_mels, int(chunk_s * 16000)

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        wav = ni.tensor_inputs["audio"][0].float().reshape(-1)
        n = max(1, -(-wav.numel() // self.chunk))
        wav = torch.nn.functional.pad(wav, (0, n * self.chunk - wav.numel())).reshape(n, self.chunk).to(self.device)
        feats, _ = self.enc([log_mel_spectrogram(w, n_mels=self.n_mels) for w in wav])
        return {"audio_features": feats}


def frames_per_chunk(chunk_s: float = CHUNK_S) -> int:
    return int(chunk_s * 16000) // 160 // 2        # hop 160, conv stride 2


class HiggsAudioModel(Model):
    name = "higgs_audio"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        if small:
            k = small_scale()
            self.cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                                     intermediate_size=128 * k, vocab_size=151936, qk_norm=True, tie_embeddings=True, dtype=dt)
            self.enc_cfg, self.n_mels = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, dtype=dt), 16
        else:      # Qwen3-1.7B backbone
            self.cfg = DecoderConfig(hidden_size=2048, num_layers=28, num_heads=16, num_kv_heads=8, head_dim=128,
                                     intermediate_size=6144, vocab_size=151936, qk_norm=True, tie_embeddings=True,
                                     rope_theta=1e6, dtype=dt)
            self.enc_cfg, self.n_mels = EncoderConfig(1280, 32, 20, 64, 5120, dtype=dt), 128
        self.sm = LMStateMachine()

    def get_graph_walk_graphs(self):
        enc = GraphNode("audio_encoder", {"audio"}, [GraphEdge("LLM", "audio_features")])
        text = lm_walks()
        audio = lm_walks(prefill_inputs={"audio_features"}, pre_nodes=[enc])
        return {"prefill_text": text["prefill"], "prefill_audio": audio["prefill"], "decode": text["decode"]}

    def get_node_engine_types(self):
        return {"audio_encoder": EngineType.STATELESS, "LLM": EngineType.KV_CACHE}

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=32768,
                              max_num_pages=64 if self.small else 2048, page_size=16 if self.small else 128,
                              num_qo_heads=c.num_heads, nodes=["LLM"], dtype=c.dtype)]

    def get_engine_hints(self, node):
        return dict(vocab_size=self.cfg.vocab_size, group=self.cfg.num_heads // self.cfg.num_kv_heads,
                    max_tokens=32768, track_seen=False)

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "audio_encoder":
            enc = AudioEncoder(self.enc_cfg, n_mels=self.n_mels, max_frames=frames_per_chunk(),
                               out_dim=self.cfg.hidden_size, device=device).init_random(0)
            return ChunkedAudioEncoderSubmodule(enc, device, self.n_mels)
        if node_name == "LLM":
            lm = DecoderLM(self.cfg, tp=tp_group, device=device)
            if self.skip_weight_loading or self.model_dir is None:
                lm.init_random(0)
            else:
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir, strict=False)    # layout not checked against a published file
            return MultimodalDecoderSubmodule(lm, device, {"audio_features": AUDIO_TOKEN}, eos_ids=(EOS,))
        raise KeyError(node_name)

    def get_sampling_config(self, model_kwargs):
        mk = dict(model_kwargs)
        mk.setdefault("temperature", 0.0)
        return super().get_sampling_config(mk)

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 512))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        text = self.encode_text(self.chat_text(prompt or "Transcribe the audio."), self.cfg.vocab_size, 256)
        ids = [b % 1000 for b in text]
        out = {}
        if tensors.get("audio"):
            wav = tensors["audio"][0].float().reshape(-1)
            n_chunks = max(1, -(-wav.numel() // int(CHUNK_S * 16000)))
            ids = ids + [AUDIO_BOS] + [AUDIO_TOKEN] * (n_chunks * frames_per_chunk()) + [AUDIO_EOS]
            out["audio"] = [wav]
        out["input_ids"] = [torch.tensor(ids, dtype=torch.int64)]
        return out

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        fpa = self.sm.initial(input_signals, self.get_max_output_tokens(model_kwargs),
                              [GraphEdge("audio_encoder", "audio", list(input_signals["audio"]))]
                              if input_signals.get("audio") else [])
        fpa.full_metadata["graph_walk"] = "prefill_audio" if input_signals.get("audio") else "prefill_text"
        return fpa

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = dict(partition_metadata)
        if md["finished_walk"].startswith("prefill"):
            md["finished_walk"] = "prefill"
        return self.sm.next(md, persist_signals)

    def postprocess(self, output, modality, request_kwargs):
        return self.decode_text(output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output))
