"""Qwen3-Omni-30B-A3B class any-to-text-and-speech model.

Nodes: ``audio_encoder`` / ``vision_encoder`` (stateless), ``Thinker`` (KV-cache engine; MoE decoder with 128
experts, top-8, 3-axis interleaved rotary positions), ``Talker`` (KV-cache engine; MoE decoder with a shared
expert + code predictor), ``Code2Wav`` (stateless codec).
Partitions: ``thinker`` -> ``talker`` over the stream ``thinker_out`` (one hidden state per thinker step; the
talker consumes one per frame and keeps speaking after the thinker's end), ``talker`` -> ``code2wav`` over
``codec_frames`` with left-context chunks.
Walks: ``prefill_text`` / ``prefill_audio`` / ``prefill_vision`` / ``prefill_mm`` (encoders, then ONE packed
prefill with encoder rows spliced in at placeholder tokens), ``thinker_decode``, ``talker_prefill``,
``talker_decode``, ``code2wav_chunk``.
Expert weights are cut either by column (tensor parallel) or by expert over the same group
(``moe_expert_parallel``), both summed by the row-parallel all-reduce.

Reference counterparts: mstar/model/qwen3_omni/qwen3_omni_model.py (walks :194-420, partitions :426-477, TP
:1206-1220, per-expert weight fuse :1297-1347), submodules.py (2028), components/thinker.py (259), talker.py
(549), code2wav.py (535), rope.py (368), config.py (545).
"""
from __future__ import annotations

import torch

from ..api_server.media_io import float_to_pcm16
from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop
from ..streaming import (Connection, FixedChunkPolicy, LeftContextChunkPolicy, PartitionDefinition, PartitionTopology,
                         StreamingGraphEdge)
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .code2wav import OmniCode2Wav
from .decoder import DecoderConfig, DecoderLM
from .encoders import EncoderConfig, log_mel_spectrogram
from .qwen3_omni_encoders import OmniAudioEncoder, OmniVisionEncoder, audio_output_length
from .llm_common import MultimodalDecoderSubmodule, expand_placeholders, lm_walks
from .qwen3_tts import CodecChunkSubmodule, talker_walks
from .submodule_base import NodeSubmodule
from .talker import CodePredictor, TalkerSubmodule

AUDIO_TOKEN, IMAGE_TOKEN, VISION_BOS, VISION_EOS, AUDIO_BOS, AUDIO_EOS = 151675, 151655, 151652, 151653, 151669, 151670
IM_END, ENDOFTEXT = 151645, 151643


def thinker_config(dtype, small=False, expert_parallel=False) -> DecoderConfig:
    if small:
        k = small_scale()
        return DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                             intermediate_size=128 * k, vocab_size=151936, qk_norm=True,
                             mrope_sections=[2 * k, 3 * k, 3 * k], num_experts=4,
                             num_experts_per_tok=2, moe_intermediate_size=32 * k, moe_expert_parallel=expert_parallel, dtype=dtype)
    return DecoderConfig(hidden_size=2048, num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128,
                         intermediate_size=768, vocab_size=151936, rope_theta=1e6, qk_norm=True,
                         mrope_sections=[24, 20, 20], mrope_interleaved=True, num_experts=128, num_experts_per_tok=8,
                         moe_intermediate_size=768, norm_topk_prob=True, moe_expert_parallel=expert_parallel, dtype=dtype)


def talker_config(dtype, small=False, expert_parallel=False) -> DecoderConfig:
    if small:
        k = small_scale()
        return DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                             intermediate_size=128 * k, vocab_size=128, qk_norm=True, num_experts=4,
                             num_experts_per_tok=2, moe_intermediate_size=32 * k,
                             shared_expert_intermediate_size=64 * k, moe_expert_parallel=expert_parallel, dtype=dtype)
    return DecoderConfig(hidden_size=1024, num_layers=20, num_heads=16, num_kv_heads=2, head_dim=128,
                         intermediate_size=384, vocab_size=3072, rope_theta=1e6, qk_norm=True, num_experts=128,
                         num_experts_per_tok=6, moe_intermediate_size=384, shared_expert_intermediate_size=768,
                         moe_expert_parallel=expert_parallel, dtype=dtype)


class AudioFeatureSubmodule(NodeSubmodule):
    def __init__(self, enc: OmniAudioEncoder, device, n_mels: int):
        super().__init__(device, enc.c.dtype)
        self.enc, self.n_mels = enc, n_mels

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        mels = [log_mel_spectrogram(w.float().reshape(-1).to(self.device), n_mels=self.n_mels)
                for w in ni.tensor_inputs["audio"]]
        feats, _ = self.enc(mels)
        return {"audio_features": feats}


class VisionFeatureSubmodule(NodeSubmodule):
    """Rows of ``image_features``: the merged patch features followed by the features of every tapped layer (the
    thinker adds those to its first layers' outputs at the image rows)."""

    def __init__(self, enc: OmniVisionEncoder, device):
        super().__init__(device, enc.c.dtype)
        self.enc = enc

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        imgs = [t.to(self.device) for t in ni.tensor_inputs.get("image", []) + ni.tensor_inputs.get("video", [])]
        feats, deep, _, _ = self.enc(imgs)
        return {"image_features": torch.cat([feats] + deep, dim=-1) if deep else feats}


def audio_rows(n_samples: int) -> int:
    """Rows the audio tower gives for a 16 kHz waveform (one mel frame per 160 samples)."""
    return max(1, audio_output_length(n_samples // 160))


def mrope_positions(ids: torch.Tensor, grids: list[tuple[int, int, int]], image_token: int):
    """3-axis positions for a prompt with image spans: text tokens advance all three axes together; the tokens of
    an image span take (t, h, w) offsets from the span's start; the text after a span resumes at the largest
    position used so far + 1. Returns (int32 [3, T], delta) with delta = next position - T."""
    T = ids.numel()
    pos = torch.zeros((3, T), dtype=torch.int32)
    is_img = (ids == image_token).tolist()
    nxt, i, g = 0, 0, 0
    while i < T:
        if is_img[i] and g < len(grids):
            t, h, w = grids[g]
            n = t * h * w
            tt = torch.arange(t).repeat_interleave(h * w)
            hh = torch.arange(h).repeat_interleave(w).repeat(t)
            ww = torch.arange(w).repeat(t * h)
            span = torch.stack([tt, hh, ww]).to(torch.int32) + nxt
            m = min(n, T - i)
            pos[:, i:i + m] = span[:, :m]
            nxt = int(span.max()) + 1
            i += m
            g += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - T


class Qwen3OmniModel(Model):
    name = "qwen3_omni"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, expert_parallel: bool = False,
                 max_num_pages: int | None = None, fp8_experts: bool = False, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        # block-scaled e4m3 expert weights (1 x 128 activation / 128 x 128 weight scales) in the thinker and talker
        self.fp8_experts = fp8_experts
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        self.t_cfg = thinker_config(dt, small, expert_parallel)
        self.k_cfg = talker_config(dt, small, expert_parallel)
        if small:
            k = small_scale()
            self.pred_cfg = DecoderConfig(hidden_size=32 * k, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16 * k,
                                          intermediate_size=64 * k, vocab_size=8, qk_norm=True, dtype=dt)
            self.n_sub, self.codebook, self.codec_eos = 3, 64, 63
            self.a_cfg, self.n_mels = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, act="gelu_erf", eps=1e-5, dtype=dt), 16
            self.v_cfg, self.patch, self.merge = EncoderConfig(32 * k, 2, 2, 16 * k, 64 * k, dtype=dt), 4, 2
            self.a_kw = dict(conv_channels=8, max_positions=64)
            self.v_kw = dict(pos_grid=6, deepstack=(0, 1))
            self.chunk, self.left = 6, 2
        else:
            self.pred_cfg = DecoderConfig(hidden_size=1024, num_layers=5, num_heads=16, num_kv_heads=8, head_dim=64,
                                          intermediate_size=3072, vocab_size=8, qk_norm=True, dtype=dt)
            self.n_sub, self.codebook, self.codec_eos = 15, 2048, 2150
            self.a_cfg, self.n_mels = EncoderConfig(1280, 32, 20, 64, 5120, act="gelu_erf", eps=1e-5, dtype=dt), 128
            self.v_cfg, self.patch, self.merge = EncoderConfig(1152, 27, 16, 72, 4304, dtype=dt), 16, 2
            self.a_kw = dict(conv_channels=480, max_positions=1500)
            self.v_kw = dict(pos_grid=48, deepstack=(8, 16, 24))
            self.chunk, self.left = 300, 25
        self.max_num_pages = max_num_pages or (64 if small else 2048)

    # ---- structure ----
    def get_graph_walk_graphs(self):
        a = GraphNode("audio_encoder", {"audio"}, [GraphEdge("Thinker", "audio_features")])
        v = GraphNode("vision_encoder", {"image"}, [GraphEdge("Thinker", "image_features")])
        stream = StreamingGraphEdge("Talker", "thinker_out", target_partition="talker")
        kw = dict(node="Thinker", loop_name="thinker_loop", stream_edge=stream)
        walks = {"prefill_text": lm_walks(**kw)["prefill"],
                 "prefill_audio": lm_walks(prefill_inputs={"audio_features"}, pre_nodes=[a], **kw)["prefill"],
                 "prefill_vision": lm_walks(prefill_inputs={"image_features"}, pre_nodes=[v], **kw)["prefill"],
                 "prefill_mm": lm_walks(prefill_inputs={"audio_features", "image_features"}, pre_nodes=[a, v], **kw)["prefill"],
                 "thinker_decode": lm_walks(**kw)["decode"]}
        frames = StreamingGraphEdge("Code2Wav", "codec_frames", target_partition="code2wav")
        walks.update(talker_walks("Talker", "talker_loop", "thinker_out", frames, {"thinker_out"}, count_tokens=False))
        c2w = GraphNode("Code2Wav", {"codec_frames"}, [GraphEdge(EMIT_TO_CLIENT, "audio", output_modality="audio")],
                        streaming_inputs={"codec_frames"})
        walks["code2wav_chunk"] = Loop(c2w, max_iters=1 << 20, name="code2wav_loop")
        return walks

    def get_node_engine_types(self):
        return {"audio_encoder": EngineType.STATELESS, "vision_encoder": EngineType.STATELESS,
                "Thinker": EngineType.KV_CACHE, "Talker": EngineType.KV_CACHE, "Code2Wav": EngineType.STATELESS}

    def get_partition_topology(self):
        return PartitionTopology(["thinker", "talker", "code2wav"], [
            Connection("thinker", "talker", "thinker_out", lambda: FixedChunkPolicy(1, continue_after_done=True)),
            Connection("talker", "code2wav", "codec_frames", lambda: LeftContextChunkPolicy(self.chunk, self.left))])

    def get_partitions(self):
        return [PartitionDefinition("thinker", ["prefill_text", "prefill_audio", "prefill_vision", "prefill_mm",
                                                "thinker_decode"], "prefill_text"),
                PartitionDefinition("talker", ["talker_prefill", "talker_decode"], "talker_prefill", ["thinker"]),
                PartitionDefinition("code2wav", ["code2wav_chunk"], "code2wav_chunk", ["talker"])]

    def get_kv_cache_config(self):
        out = []
        for node, c in (("Thinker", self.t_cfg), ("Talker", self.k_cfg)):
            out.append(KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=32768,
                                     max_num_pages=self.max_num_pages, page_size=16 if self.small else 128,
                                     num_qo_heads=c.num_heads, nodes=[node], dtype=c.dtype))
        return out

    def get_default_sharding_config(self):
        return {"Thinker": {"tp": True, "sp": False}, "Talker": {"tp": True, "sp": False}}

    def get_engine_hints(self, node):
        c = self.t_cfg if node == "Thinker" else self.k_cfg
        return dict(vocab_size=c.vocab_size, group=c.num_heads // c.num_kv_heads, max_tokens=32768,
                    n_pos_axes=3 if node == "Thinker" else 1, track_seen=True, max_batch=32)

    def get_autocast_dtype(self):
        return self.dtype

    def _position_fn(self, ids, inputs, kwargs):
        grids = []
        for im in inputs.get("image_grid", []):
            grids += [tuple(int(x) for x in row) for row in im.reshape(-1, 3).tolist()]
        return mrope_positions(ids, grids, IMAGE_TOKEN)

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        load = not (self.skip_weight_loading or self.model_dir is None)
        if node_name == "audio_encoder":
            enc = OmniAudioEncoder(self.a_cfg, n_mels=self.n_mels, out_dim=self.t_cfg.hidden_size, n_window=50,
                                   n_window_infer=800, device=device, **self.a_kw).init_random(0)
            if load:
                from .checkpoints import load_qwen3_omni_audio
                load_qwen3_omni_audio(enc, self.model_dir)
            return AudioFeatureSubmodule(enc, device, self.n_mels)
        if node_name == "vision_encoder":
            enc = OmniVisionEncoder(self.v_cfg, patch=self.patch, temporal_patch=2, merge=self.merge,
                                    out_dim=self.t_cfg.hidden_size, device=device, **self.v_kw).init_random(0)
            if load:
                from .checkpoints import load_qwen3_omni_vision
                load_qwen3_omni_vision(enc, self.model_dir)
            return VisionFeatureSubmodule(enc, device)
        if node_name == "Thinker":
            lm = DecoderLM(self.t_cfg, tp=tp_group, device=device)
            if load:
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir, prefix="thinker.model.", head_name="thinker.lm_head.weight")
            else:
                lm.init_random(0)
            if self.fp8_experts:
                lm.quantize_moe_fp8()
            return MultimodalDecoderSubmodule(lm, device, {"audio_features": AUDIO_TOKEN, "image_features": IMAGE_TOKEN},
                                              eos_ids=(IM_END, ENDOFTEXT), loop_name="thinker_loop",
                                              position_fn=self._position_fn, emit_hidden="thinker_out",
                                              deepstack={"image_features": len(self.v_kw["deepstack"])})
        if node_name == "Talker":
            lm = DecoderLM(self.k_cfg, tp=tp_group, device=device)
            if load:
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir, prefix="talker.model.", head_name="talker.codec_head.weight",
                                     embed_name="codec_embedding.weight")
            else:
                lm.init_random(2)
            if self.fp8_experts:
                lm.quantize_moe_fp8()
            pred = CodePredictor(self.pred_cfg, self.k_cfg.hidden_size, self.n_sub, self.codebook, device).init_random(3)
            if load:
                from .checkpoints import load_qwen3_omni_code_predictor
                load_qwen3_omni_code_predictor(pred, self.model_dir)
            return TalkerSubmodule(lm, pred, device, num_slots=64, codec_eos=self.codec_eos, cond_edge="thinker_out",
                                   cond_is_ids=False, cond_dim=self.t_cfg.hidden_size, loop_name="talker_loop",
                                   suppress_from=self.codebook)
        if node_name == "Code2Wav":
            k = small_scale()
            kw = (dict(n_codebooks=self.n_sub + 1, codebook_size=self.codebook, hidden=32 * k, layers=1, heads=2,
                       head_dim=16 * k, ffn=64 * k, window=4, upsampling_ratios=(2,), upsample_rates=(2,), decoder_dim=16 * k)
                  if self.small else {})                   # the published shapes are the defaults
            dec = OmniCode2Wav(dtype=self.dtype, device=device, **kw).init_random(5)
            if load:
                from .checkpoints import load_qwen3_omni_code2wav
                load_qwen3_omni_code2wav(dec, self.model_dir)
            return CodecChunkSubmodule(dec.eval(), device, "codec_frames", self.left, "code2wav_loop")
        raise KeyError(node_name)

    # ---- request life cycle ----
    @staticmethod
    def _audio_budget(model_kwargs) -> int:
        """Upper bound of codec frames per request (the talker normally stops at its end-of-speech code)."""
        return int((model_kwargs or {}).get("max_audio_tokens", 4096))

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 2048))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        v = self.t_cfg.vocab_size
        ids = self.encode_text(self.chat_text(prompt), v, 1000)
        out = {}
        if tensors.get("audio"):
            wavs = [w.float().reshape(-1) for w in tensors["audio"]]
            for w in wavs:
                ids += [AUDIO_BOS] + [AUDIO_TOKEN] * audio_rows(w.numel()) + [AUDIO_EOS]
            out["audio"] = wavs
        if tensors.get("image"):
            imgs, grids = [], []
            for im in tensors["image"]:
                im = im.float()
                C, H, W = im.shape[0], im.shape[-2], im.shape[-1]
                t = 1 if im.dim() == 3 else im.shape[1] // 2
                h, w = H // self.patch // self.merge, W // self.patch // self.merge
                ids += [VISION_BOS] + [IMAGE_TOKEN] * (t * h * w) + [VISION_EOS]
                grids.append([t, h, w])
                imgs.append(im)
            out["image"], out["image_grid"] = imgs, [torch.tensor(grids, dtype=torch.int64)]
        out["input_ids"] = [torch.tensor([i % v for i in ids] or [0], dtype=torch.int64)]
        return out

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        speak = "audio" in (output_modalities or [])
        if partition_name == "talker":
            return ForwardPassArgs({"graph_walk": "talker_prefill", "max_tokens": self._audio_budget(model_kwargs)},
                                   []) if speak else None
        if partition_name == "code2wav":
            return ForwardPassArgs({"graph_walk": "code2wav_chunk"}, []) if speak else None
        a, i = bool(input_signals.get("audio")), bool(input_signals.get("image"))
        walk = "prefill_mm" if a and i else "prefill_audio" if a else "prefill_vision" if i else "prefill_text"
        edges = [GraphEdge("Thinker", "input_ids", list(input_signals["input_ids"]))]
        if a:
            edges.append(GraphEdge("audio_encoder", "audio", list(input_signals["audio"])))
        if i:
            edges.append(GraphEdge("vision_encoder", "image", list(input_signals["image"])))
            edges.append(GraphEdge("Thinker", "image_grid", list(input_signals["image_grid"])))
        return ForwardPassArgs({"graph_walk": walk, "max_tokens": self.get_max_output_tokens(model_kwargs)}, edges)

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        if partition_name == "code2wav":
            return ForwardPassArgs(request_done=True)
        node, walk, loop = (("Talker", "talker_decode", "talker_loop") if partition_name == "talker"
                            else ("Thinker", "thinker_decode", "thinker_loop"))
        budget = (self._audio_budget(md.get("model_kwargs")) if partition_name == "talker"
                  else md["max_tokens"] - md["tokens_out"])
        if "prefill" in md["finished_walk"] and budget > 0 and persist_signals.get("last_token"):
            last = persist_signals.pop("last_token")
            return ForwardPassArgs({"graph_walk": walk, "max_tokens": budget, "dynamic_loop_iter_counts": {loop: budget}},
                                   [GraphEdge(node, "tok", last[-1:])], unpersist_tensors=[t.uuid for t in last])
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        if modality == "audio":
            return float_to_pcm16(output if isinstance(output, torch.Tensor) else torch.cat(list(output)))
        return self.decode_text(output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output))
