"""Qwen3-TTS class text-to-speech: a talker (decoder + code predictor, 16 codebooks per 12.5 Hz frame) streams
codec frames into a waveform decoder partition with left-context chunking (300 new frames, 25 frames of context).

Nodes: ``Talker`` (KV-cache engine), ``Codec`` (stateless, audio_codec flavor).
Walks: ``talker_prefill``, ``talker_decode`` (Loop ``talker_loop``), ``codec_chunk`` (Loop ``codec_loop``).
Reference counterparts: mstar/model/qwen3_tts/qwen3_tts_model.py (818 lines), submodules.py (948; piecewise graphs
:685-715), components/talker.py (316), config.py (309).
"""
from __future__ import annotations

import torch

from ..api_server.media_io import float_to_pcm16
from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop
from ..streaming import Connection, LeftContextChunkPolicy, PartitionDefinition, PartitionTopology, StreamingGraphEdge
from .base import small_scale, EngineType, ForwardPassArgs, Model, seeded_init
from .codec import Code2Wav
from .decoder import DecoderConfig, DecoderLM
from .submodule_base import NodeSubmodule
from .talker import CodePredictor, TalkerSubmodule

CODEC_EOS = 2150
N_CODEBOOKS = 16


class CodecChunkSubmodule(NodeSubmodule):
    """Frames [n, n_codebooks] -> PCM; with left context the samples that belong to the context frames are cut."""

    def __init__(self, dec: Code2Wav, device, edge: str, left_context: int, loop_name: str):
        super().__init__(device, torch.float32)
        self.dec, self.edge, self.left, self.loop_name = dec, edge, left_context, loop_name

    def get_stateless_flavor(self):
        return "audio_codec"

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        fr = ni.tensor_inputs.get(self.edge, [])
        st = engine_inputs.per_request_states[ni.request_id]
        final = bool(ni.kwargs.get("final_chunk"))
        if not fr:
            return {"audio": torch.zeros(0), "final": final}
        codes = torch.cat([t.reshape(-1, t.shape[-1]) for t in fr]).to(self.device).long()      # [n, K]
        with torch.no_grad():
            wav = self.dec(codes.t()[None].contiguous())[0]
        ctx = self.left if st.get("seen_first") else 0
        st["seen_first"] = True
        return {"audio": wav[min(ctx, codes.shape[0]) * self.dec.hop:].float().cpu(), "final": final}

    def postprocess(self, request_id, request_info, outputs, inputs):
        return {"audio": outputs["audio"]}

    def check_stop(self, request_id, request_info, outputs):
        return {self.loop_name} if outputs.get("final") or (request_info.step_metadata or {}).get("final_chunk") else set()


def talker_walks(node: str, loop: str, cond_edge: str | None, frame_stream: StreamingGraphEdge,
                 prefill_inputs: set[str], max_iters: int = 4096, count_tokens: bool = True) -> dict:
    """``count_tokens``: the talker's codes count toward the request's output-token budget (a TTS model); off when
    another partition produces the budgeted tokens (the thinker of an omni model)."""
    def outs(extra):
        return [GraphEdge(EMPTY_DESTINATION, "new_token", conductor_new_token=count_tokens), frame_stream.clone()] + extra
    pre = GraphNode(node, set(prefill_inputs), [GraphEdge(EMPTY_DESTINATION, "new_token", conductor_new_token=count_tokens),
                                                GraphEdge(EMPTY_DESTINATION, "last_token", persist=True)],
                    streaming_inputs={cond_edge} & set(prefill_inputs) if cond_edge else set())
    ins = {"tok"} | ({cond_edge} if cond_edge else set())
    step = GraphNode(node, ins, outs([GraphEdge(node, "tok")]), streaming_inputs={cond_edge} if cond_edge else set())
    return {"talker_prefill": pre, "talker_decode": Loop(step, max_iters=max_iters, name=loop)}


class Qwen3TTSModel(Model):
    name = "qwen3_tts"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        if small:
            k = small_scale()
            self.cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                                     intermediate_size=128 * k, vocab_size=3072, qk_norm=True, dtype=dt)
            self.pred_cfg = DecoderConfig(hidden_size=32 * k, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16 * k,
                                          intermediate_size=64 * k, vocab_size=8, qk_norm=True, dtype=dt)
            self.n_sub, self.codebook, self.text_vocab = 3, 64, 512
            self.chunk, self.left = 6, 2
        else:     # 1.7B-class talker, 5-layer predictor
            self.cfg = DecoderConfig(hidden_size=2048, num_layers=28, num_heads=16, num_kv_heads=8, head_dim=128,
                                     intermediate_size=6144, vocab_size=3072, qk_norm=True, rope_theta=1e6, dtype=dt)
            self.pred_cfg = DecoderConfig(hidden_size=1024, num_layers=5, num_heads=16, num_kv_heads=8, head_dim=64,
                                          intermediate_size=3072, vocab_size=8, qk_norm=True, dtype=dt)
            self.n_sub, self.codebook, self.text_vocab = N_CODEBOOKS - 1, 2048, 151936
            self.chunk, self.left = 300, 25
        self.codec_eos = CODEC_EOS if not small else 63

    def get_graph_walk_graphs(self):
        stream = StreamingGraphEdge("Codec", "codec_frames", target_partition="codec")
        walks = talker_walks("Talker", "talker_loop", None, stream, {"text_ids"})
        codec = GraphNode("Codec", {"codec_frames"}, [GraphEdge(EMIT_TO_CLIENT, "audio", output_modality="audio")],
                          streaming_inputs={"codec_frames"})
        walks["codec_chunk"] = Loop(codec, max_iters=1 << 20, name="codec_loop")
        return walks

    def get_node_engine_types(self):
        return {"Talker": EngineType.KV_CACHE, "Codec": EngineType.STATELESS}

    def get_partition_topology(self):
        return PartitionTopology(["talker", "codec"], [Connection("talker", "codec", "codec_frames",
                                                                  lambda: LeftContextChunkPolicy(self.chunk, self.left))])

    def get_partitions(self):
        return [PartitionDefinition("talker", ["talker_prefill", "talker_decode"], "talker_prefill"),
                PartitionDefinition("codec", ["codec_chunk"], "codec_chunk", ["talker"])]

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=8192,
                              max_num_pages=64 if self.small else 2048, page_size=16 if self.small else 128,
                              num_qo_heads=c.num_heads, nodes=["Talker"], dtype=c.dtype)]

    def get_engine_hints(self, node):
        return dict(vocab_size=self.cfg.vocab_size, group=self.cfg.num_heads // self.cfg.num_kv_heads,
                    max_tokens=8192, track_seen=True, max_batch=32)

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "Talker":
            lm = DecoderLM(self.cfg, tp=tp_group, device=device).init_random(0)
            pred = CodePredictor(self.pred_cfg, self.cfg.hidden_size, self.n_sub, self.codebook, device).init_random(1)
            if not (self.skip_weight_loading or self.model_dir is None):
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir, prefix="talker.model.", head_name="talker.codec_head.weight",
                                     strict=False)       # this checkpoint layout has not been checked against a published file
            return TalkerSubmodule(lm, pred, device, num_slots=64, codec_eos=self.codec_eos, cond_edge="text_ids",
                                   cond_is_ids=True, cond_dim=0, loop_name="talker_loop", text_vocab=self.text_vocab)
        if node_name == "Codec":
            kw = (dict(n_codebooks=self.n_sub + 1, codebook_size=self.codebook, dim=16, rates=(2, 2), channels=32)
                  if self.small else dict(n_codebooks=N_CODEBOOKS, codebook_size=2048, dim=512, rates=(8, 5, 4, 3, 4)))
            return CodecChunkSubmodule(seeded_init(lambda: Code2Wav(**kw)).to(device).eval(), device, "codec_frames", self.left, "codec_loop")
        raise KeyError(node_name)

    def get_sampling_config(self, model_kwargs):
        mk = dict(model_kwargs)
        mk.setdefault("temperature", 0.9)
        mk.setdefault("top_k", 50)
        mk.setdefault("repetition_penalty", 1.05)
        return super().get_sampling_config(mk)

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 2048))

    def get_output_sample_rate(self):
        return 24000

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        ids = self.encode_text(prompt, self.text_vocab, default=" ")
        return {"text_ids": [torch.tensor(ids, dtype=torch.int64)]}

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        if partition_name == "codec":
            return ForwardPassArgs({"graph_walk": "codec_chunk"}, [])
        return ForwardPassArgs({"graph_walk": "talker_prefill", "max_tokens": self.get_max_output_tokens(model_kwargs)},
                               [GraphEdge("Talker", "text_ids", list(input_signals["text_ids"]))])

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        if partition_name == "codec":
            return ForwardPassArgs(request_done=True)
        budget = md["max_tokens"] - md["tokens_out"]
        if md["finished_walk"] == "talker_prefill" and budget > 0 and persist_signals.get("last_token"):
            last = persist_signals.pop("last_token")
            return ForwardPassArgs({"graph_walk": "talker_decode", "max_tokens": budget,
                                    "dynamic_loop_iter_counts": {"talker_loop": budget}},
                                   [GraphEdge("Talker", "tok", last[-1:])], unpersist_tensors=[t.uuid for t in last])
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        return float_to_pcm16(output if isinstance(output, torch.Tensor) else torch.cat(list(output)))
