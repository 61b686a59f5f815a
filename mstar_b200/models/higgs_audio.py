"""Higgs-Audio v3 class speech-to-text in the published layout: a Whisper-style audio tower over 4-second chunks
(two convolutions, position table, pre-LN transformer, average pooling by 2, final LayerNorm: 25 rows per second), a
projector (depthwise stride-2 convolution over time, then a two-layer ReLU MLP: 12.5 rows per second) and a dense
Qwen3-1.7B class decoder that takes the projected rows at its audio placeholder tokens.

Chunks are padded to the longest one and each is its own attention sequence; the rows of a chunk beyond its valid
length are dropped after the projector. Walks: ``prefill_text`` (no audio), ``prefill_audio`` (tower, projector, then
one packed prefill), ``decode``.
Reference counterparts: mstar/model/higgs_audio/higgs_audio_model.py (519 lines), submodules.py (218),
components/audio_tower.py (tower :27-63, projector :66-87), config.py (token ids :38-43, row count :64-69).
"""
from __future__ import annotations

import torch
from torch import nn

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import GraphEdge, GraphNode
from ..ops import gemm
from .base import small_scale, EngineType, Model
from .decoder import DecoderConfig, DecoderLM
from .encoders import AudioEncoder, EncoderConfig, log_mel_spectrogram
from .llm_common import LMStateMachine, MultimodalDecoderSubmodule, lm_walks
from .submodule_base import NodeSubmodule

AUDIO_TOKEN, AUDIO_BOS, AUDIO_EOS, IM_END, EOS = 151672, 151669, 151670, 151645, 151643
CHUNK_S, HOP, MIN_SAMPLES = 4.0, 160, 1600
DEFAULT_PROMPT = "Transcribe the speech. Output only the spoken words in lowercase with no punctuation."


def audio_rows(n_samples: int) -> int:
    """Decoder rows of a chunk of ``n_samples``: mel frames -> stride-2 convolution -> pooling by 2 -> stride-2
    projector convolution."""
    mel = -(-n_samples // HOP)
    conv = (mel - 1) // 2 + 1
    pooled = (conv - 2) // 2 + 1
    return max(0, (pooled - 1) // 2 + 1)


def chunk_lengths(n_samples: int, chunk: int = int(CHUNK_S * 16000)) -> list[int]:
    n = max(n_samples, 1)
    return [min(chunk, n - i) for i in range(0, n, chunk)]


class AudioProjector(nn.Module):
    """Depthwise Conv1d(k 3, stride 2, padding 1) over the rows of each chunk, then Linear -> ReLU -> Linear."""

    def __init__(self, dim: int, mid: int, out_dim: int, dtype, device):
        super().__init__()
        self.temporal = nn.Conv1d(dim, dim, 3, 2, padding=1, groups=dim).to(device=device, dtype=dtype)
        def P(*shape):
            return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)
        self.w1, self.b1, self.w2, self.b2 = P(mid, dim), P(mid), P(out_dim, mid), P(out_dim)
        for p in self.temporal.parameters():
            p.requires_grad_(False)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for p in self.parameters():
            if p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g) / (p[0].numel() ** 0.5)).to(p.dtype))
        return self

    def forward(self, x: torch.Tensor, lens: list[int]) -> tuple[torch.Tensor, list[int]]:
        """x: packed rows [sum lens, dim] -> packed rows [sum ceil(len / 2), out_dim]."""
        parts = [self.temporal(h.transpose(0, 1)[None])[0].transpose(0, 1) for h in x.split(lens)]
        out = [h.shape[0] for h in parts]
        h = torch.relu(gemm.linear(torch.cat(parts).contiguous(), self.w1, self.b1))
        return gemm.linear(h, self.w2, self.b2), out


class ChunkedAudioEncoderSubmodule(NodeSubmodule):
    """Splits the waveform into fixed chunks, pads them with silence to the longest one, encodes them as one packed
    batch and keeps each chunk's valid rows."""

    def __init__(self, enc: AudioEncoder, proj: AudioProjector, device, n_mels: int, chunk_s: float = CHUNK_S):
        super().__init__(device, enc.c.dtype)
        self.enc, self.proj, self.n_mels, self.chunk = enc, proj, n_mels, int(chunk_s * 16000)

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        wav = ni.tensor_inputs["audio"][0].float().reshape(-1).to(self.device)
        lens = chunk_lengths(wav.numel(), self.chunk)
        longest = max(max(lens), MIN_SAMPLES)
        mels, at = [], 0
        for n in lens:
            mels.append(log_mel_spectrogram(torch.nn.functional.pad(wav[at:at + n], (0, longest - n)), n_mels=self.n_mels))
            at += n
        feats, rows = self.enc(mels)
        feats, rows = self.proj(feats, rows)
        keep = [h[:min(audio_rows(n), h.shape[0])] for h, n in zip(feats.split(rows), lens)]
        return {"audio_features": torch.cat(keep).contiguous()}


def placeholder_rows(n_samples: int) -> int:
    """Audio placeholder tokens of a waveform: what ``ChunkedAudioEncoderSubmodule`` emits for it."""
    lens = chunk_lengths(n_samples)
    longest = max(max(lens), MIN_SAMPLES)
    cap = audio_rows(longest // HOP * HOP)            # rows the padded chunk yields
    return sum(min(audio_rows(n), cap) for n in lens)


LM_HEAD = "audio_decoder_proj.text_lm_head.weight"


def llm_checkpoint_name(name: str) -> str | None:
    """Names of the decoder's tensors in the published file: the tower, the projector and the speech-generation parts
    (codebook embeddings, audio heads) are not the decoder's; the text head sits beside the audio heads."""
    if name == LM_HEAD:
        return name
    if name.startswith(("audio_tower.", "audio_encoder_proj.", "audio_codebook_embeddings.", "audio_decoder_proj.")):
        return None
    return name


class HiggsAudioModel(Model):
    name = "higgs_audio"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        if small:
            k = small_scale()
            self.cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                                     intermediate_size=128 * k, vocab_size=151936, qk_norm=True, tie_embeddings=False, dtype=dt)
            self.enc_cfg = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, act="gelu_erf", eps=1e-5, dtype=dt)
            self.n_mels, self.proj_mid = 16, 64 * k
        else:      # Qwen3-1.7B backbone with its own output head; Whisper-large-v3 sized tower
            self.cfg = DecoderConfig(hidden_size=2048, num_layers=28, num_heads=16, num_kv_heads=8, head_dim=128,
                                     intermediate_size=6144, vocab_size=151936, qk_norm=True, tie_embeddings=False,
                                     rope_theta=1e6, dtype=dt)
            self.enc_cfg = EncoderConfig(1280, 32, 20, 64, 5120, act="gelu_erf", eps=1e-5, dtype=dt)
            self.n_mels, self.proj_mid = 128, 2048
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
            enc = AudioEncoder(self.enc_cfg, n_mels=self.n_mels, max_frames=1500, device=device, pool=2)
            proj = AudioProjector(self.enc_cfg.hidden_size, self.proj_mid, self.cfg.hidden_size, self.dtype, device)
            if self.skip_weight_loading or self.model_dir is None:
                enc.init_random(0)
                proj.init_random(1)
            else:
                from .checkpoints import load_higgs_audio_tower
                load_higgs_audio_tower(enc, proj, self.model_dir)
            return ChunkedAudioEncoderSubmodule(enc, proj, device, self.n_mels)
        if node_name == "LLM":
            lm = DecoderLM(self.cfg, tp=tp_group, device=device)
            if self.skip_weight_loading or self.model_dir is None:
                lm.init_random(0)
            else:
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir, head_name=LM_HEAD, layer_filter=llm_checkpoint_name)
            return MultimodalDecoderSubmodule(lm, device, {"audio_features": AUDIO_TOKEN}, eos_ids=(EOS, IM_END))
        raise KeyError(node_name)

    def get_sampling_config(self, model_kwargs):
        mk = dict(model_kwargs)
        mk.setdefault("temperature", 0.0)
        return super().get_sampling_config(mk)

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 512))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        """ChatML user turn: the instruction, then the audio rows between the audio begin / end tokens, then the
        assistant header (with an empty think block unless ``enable_thinking``). Without the checkpoint's tokenizer
        the text parts are byte-level ids."""
        prompt = prompt or DEFAULT_PROMPT
        out, audio = {}, []
        if tensors.get("audio"):
            if len(tensors["audio"]) != 1:
                raise ValueError(f"one audio input per request, got {len(tensors['audio'])}")
            wav = tensors["audio"][0].float().reshape(-1)
            audio = [AUDIO_BOS] + [AUDIO_TOKEN] * placeholder_rows(wav.numel()) + [AUDIO_EOS]
            out["audio"] = [wav]
        tok = self.tokenizer()
        if tok is not None:
            def enc(t):
                return list(tok.encode(t, add_special_tokens=False))
            post = "<|im_end|>\n<|im_start|>assistant\n" + ("" if kw.get("enable_thinking") else "<think>\n\n</think>\n\n")
            ids = enc("<|im_start|>user\n") + enc(prompt) + audio + enc(post)
        else:
            ids = [b % 1000 for b in self.encode_text(self.chat_text(prompt), self.cfg.vocab_size, 256)] + audio
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
