"""Orpheus-3B TTS: Llama-3.2-3B backbone that emits audio tokens, and a SNAC-style codec decoder fed through a
sliding-window stream (window 28 tokens = 4 frames, stride 7 = 1 frame); every chunk yields the second frame's
2048 samples.

Nodes: ``LLM`` (KV-cache engine, tensor-parallel capable), ``snac_decoder`` (stateless, audio_codec flavor, fp32).
Partitions: ``llm`` (walks prefill, decode) -> ``codec`` (walk snac_chunk) over the streaming edge ``audio_tokens``.

Reference counterparts: mstar/model/orpheus/orpheus_model.py (walks :111-167, partitions :173-203, state machine
:205-281, TP defaults :406-409), submodules.py, components/{language_model,snac}.py, config.py.
"""
from __future__ import annotations

import os

import torch

from ..api_server.media_io import float_to_pcm16
from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, GraphEdge, GraphNode, Loop
from ..streaming import Connection, PartitionDefinition, PartitionTopology, SlidingWindowChunkPolicy, StreamingGraphEdge
from .base import EngineType, ForwardPassArgs, Model, seeded_init
from .codec import SnacDecoder, orpheus_tokens_to_codes
from .decoder import DecoderConfig, DecoderLM
from .llm_common import DecoderSubmodule, LMStateMachine, lm_walks
from .orpheus_config import orpheus_3b_config
from .submodule_base import NodeSubmodule
from ..utils import io_counters

CUSTOM_TOKEN_BASE = 128256
END_TOKEN_IDS = (128009, 128260, 128261, 128257, 128258)
VOICES = ["tara", "zoe", "zac", "jess", "leo", "mia", "julia", "leah"]


class _HostBatch:
    """A pinned host buffer that a queued device-to-host copy fills. The first read (after the batch's event) copies
    the used rows out ONCE; every request's waveform is then a view of that copy."""
    __slots__ = ("pinned", "rows", "copy")

    def __init__(self, pinned, rows):
        self.pinned, self.rows, self.copy = pinned, rows, None

    def get(self) -> torch.Tensor:
        if self.copy is None:
            self.copy = self.pinned[:self.rows].clone()
        return self.copy


class _HostRows:
    """One request's slice of a ``_HostBatch``."""
    __slots__ = ("batch", "row", "lo", "hi")

    def __init__(self, batch, row, lo, hi):
        self.batch, self.row, self.lo, self.hi = batch, row, lo, hi

    def get(self) -> torch.Tensor:
        return self.batch.get()[self.row, self.lo:self.hi]


class SnacSubmodule(NodeSubmodule):
    def __init__(self, device, base_id: int, small: bool, compute_dtype: torch.dtype = torch.float32,
                 snac_dir: str | None = None):
        super().__init__(device, torch.float32)
        self.compute_dtype = compute_dtype         # fp32 weights; bf16 runs the convolutions under autocast
        kw = dict(latent_dim=64, channels=64, rates=(8, 8, 4, 2)) if small else {}
        self.dec = seeded_init(lambda: SnacDecoder(**kw))
        if snac_dir:            # the published codec checkpoint (config.json + pytorch_model.bin): strict load
            from .checkpoints import load_snac_decoder
            load_snac_decoder(self.dec, snac_dir)
        self.dec = self.dec.to(device=device, dtype=torch.float32).eval()

        self.base_id = base_id
        self.gen = None
        # MSTAR_SNAC_FULL_WINDOW=1 decodes all four frames of a streaming window and slices the second one out
        self.middle_only = os.environ.get("MSTAR_SNAC_FULL_WINDOW", "0") != "1"

    def get_stateless_flavor(self):
        return "audio_codec"

    def max_batch_size(self, graph_walk):
        return 64

    @staticmethod
    def _tokens(ni) -> torch.Tensor:
        toks = ni.tensor_inputs.get("audio_tokens", [])
        t = torch.cat([x.reshape(-1) for x in toks]).cpu() if toks else torch.zeros(0, dtype=torch.int64)
        return t[:(t.numel() // 7) * 7]

    def _decode(self, tokens: torch.Tensor, runner, keep: tuple[int, int] | None = None) -> torch.Tensor:
        """tokens [B, n] (n a multiple of 7, host) -> waveforms [B, n / 7 * 2048] on the device (with ``keep`` only
        those samples, computed from their receptive field alone); replayed from a CUDA graph per shape. On a GPU the
        result is a view of the graph's static output: copy it out on the same stream."""
        def fn(tk):
            if not tk.is_cuda:
                return self.dec(orpheus_tokens_to_codes(tk, self.base_id), keep=keep)
            if self.compute_dtype != torch.float32:
                with torch.autocast("cuda", dtype=self.compute_dtype):
                    wav = self.dec(orpheus_tokens_to_codes(tk, self.base_id), keep=keep).float()
            else:
                wav = self.dec(orpheus_tokens_to_codes(tk, self.base_id), keep=keep)
            # 16-bit PCM is what leaves the server: quantise inside the captured graph, so the read-back is half
            # the bytes and the API process only forwards them
            return (wav.float().clamp(-1, 1) * 32767.0).round().to(torch.int16)
        with torch.no_grad():
            if runner is not None and self.device.type == "cuda":
                # batch padded to a power of two: a handful of captured graphs serve every batch size
                B = tokens.shape[0]
                Bp = 1 << (B - 1).bit_length()
                stage = self._pinned(("tok", Bp, tokens.shape[1]), (Bp, tokens.shape[1]), torch.int64)
                stage[:B].copy_(tokens)
                if Bp != B:
                    stage[B:] = stage[0]
                tk = stage.to(self.device, non_blocking=True)
                io_counters.add_h2d(stage.numel() * 8)
                return runner.run(("snac", tuple(tk.shape), keep), fn, [tk])[:B]
            return fn(tokens.to(self.device))

    def _pinned(self, key, shape, dtype) -> torch.Tensor:
        """Next buffer of a small ring of pinned host buffers per shape: a buffer is reused only four batches later,
        long after the copy that used it has run."""
        if not hasattr(self, "_pin"):
            self._pin = {}
        ring = self._pin.setdefault(key, [[], 0])
        if len(ring[0]) < 4:
            ring[0].append(torch.empty(shape, dtype=dtype, pin_memory=self.device.type == "cuda"))
            return ring[0][-1]
        ring[1] = (ring[1] + 1) % 4
        return ring[0][ring[1]]

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        return self.forward_batched(graph_walk, engine_inputs, [ni])[0]

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        """Requests whose chunks have the same length are decoded as one batch (streams that decode in lockstep
        hand in their 28-token windows at the same step). Nothing here waits for the GPU: the waveforms are copied
        to pinned host memory behind the decode and sliced per request in ``postprocess``, which the engine calls
        once the batch's event has passed."""
        runner = (engine_inputs.preallocated_buffers or {}).get("graph_runner")
        toks = [self._tokens(ni) for ni in inputs]
        outs: list[dict | None] = [None] * len(inputs)
        by_len: dict[tuple[int, bool], list[int]] = {}
        for i, t in enumerate(toks):
            final = bool(inputs[i].kwargs.get("final_chunk"))
            if t.numel() == 0:
                outs[i] = {"audio": torch.zeros(0), "final": final}
            else:
                # steady state: a full 4-frame window yields its second frame, and only that frame is decoded (the
                # positions its samples depend on); shorter (first / flush) windows yield everything
                by_len.setdefault((t.numel(), self.middle_only and t.numel() == 28 and not final), []).append(i)
        for (n, middle), idx in by_len.items():
            wav = self._decode(torch.stack([toks[i] for i in idx]), runner, keep=(2048, 4096) if middle else None)
            if wav.dtype != torch.int16:
                wav = wav.float()
            if wav.is_cuda:
                rows = 64 if len(idx) <= 64 else len(idx)
                host = self._pinned(("wav", rows, wav.shape[1]), (rows, wav.shape[1]), wav.dtype)
                host[:len(idx)].copy_(wav, non_blocking=True)
                io_counters.add_d2h(wav.numel() * wav.element_size())
            else:
                host = wav
            hb = _HostBatch(host, len(idx))
            for row, i in enumerate(idx):
                final = bool(inputs[i].kwargs.get("final_chunk"))
                lo, hi = (2048, 4096) if n == 28 and not final and not middle else (0, host.shape[1])
                outs[i] = {"audio": _HostRows(hb, row, lo, hi), "final": final}
        return outs

    def postprocess(self, request_id, request_info, outputs, inputs):
        a = outputs["audio"]
        return {"audio": a.get() if isinstance(a, _HostRows) else a}

    def check_stop(self, request_id, request_info, outputs):
        return {"snac_loop"} if outputs.get("final") or (request_info.step_metadata or {}).get("final_chunk") else set()


class OrpheusModel(Model):
    name = "orpheus"
    raw_payload_dtypes = {"audio": "int16"}        # the codec's graph quantises to 16-bit PCM: its bytes go out as they are

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, page_size: int = 128,
                 max_num_pages: int = 2048, codec_dtype: str = "float32", snac_dir: str | None = None, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        self.small, self.snac_dir = small, snac_dir
        self.codec_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[codec_dtype]
        if small:      # test-sized backbone with the real vocabulary layout
            self.cfg = DecoderConfig(hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                                     intermediate_size=256, vocab_size=156940, rms_eps=1e-5, rope_theta=5e5,
                                     tie_embeddings=True,
                                     dtype=torch.bfloat16 if torch.cuda.is_available() else torch.float32)
        else:
            self.cfg = orpheus_3b_config()
        self.page_size, self.max_num_pages = page_size, max_num_pages
        self.sm = LMStateMachine()

    # ---- structure ----
    def get_graph_walk_graphs(self):
        stream = StreamingGraphEdge("snac_decoder", "audio_tokens", target_partition="codec")
        walks = lm_walks(modality="", stream_edge=stream)
        snac = GraphNode("snac_decoder", {"audio_tokens"},
                         [GraphEdge(EMIT_TO_CLIENT, "audio", output_modality="audio")], streaming_inputs={"audio_tokens"})
        walks["snac_chunk"] = Loop(snac, max_iters=1 << 20, name="snac_loop")
        return walks

    def get_node_engine_types(self):
        return {"LLM": EngineType.KV_CACHE, "snac_decoder": EngineType.STATELESS}

    def get_partition_topology(self):
        return PartitionTopology(["llm", "codec"], [Connection("llm", "codec", "audio_tokens",
                                                               lambda: SlidingWindowChunkPolicy(28, 7))])

    def get_partitions(self):
        return [PartitionDefinition("llm", ["prefill", "decode"], "prefill"),
                PartitionDefinition("codec", ["snac_chunk"], "snac_chunk", ["llm"])]

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=8192 if self.small else 131072,
                              max_num_pages=self.max_num_pages, page_size=self.page_size, num_qo_heads=c.num_heads,
                              nodes=["LLM"], dtype=c.dtype)]

    def get_default_sharding_config(self):
        return {"LLM": {"tp": True, "sp": False}}

    def get_engine_hints(self, node):
        c = self.cfg
        # one audio frame (7 tokens) per node execution: the codec consumes whole frames anyway
        return dict(vocab_size=c.vocab_size, group=c.num_heads // c.num_kv_heads, max_tokens=16384, track_seen=True,
                    decode_burst=7)

    def get_autocast_dtype(self):
        return self.cfg.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "LLM":
            lm = DecoderLM(self.cfg, tp=tp_group, device=device)
            if self.skip_weight_loading:
                lm.init_random(0)
            else:
                from .loader import load_decoder_from_hf
                load_decoder_from_hf(lm, self.model_dir)
            import os
            if os.environ.get("MSTAR_FOLD_NORMS", "0") == "1":      # decode steps without norm kernels: no gain measured
                lm.fold_norms()
            return DecoderSubmodule(lm, device, eos_ids=END_TOKEN_IDS, token_edge="audio_tokens")
        if node_name == "snac_decoder":
            return SnacSubmodule(device, CUSTOM_TOKEN_BASE, self.small, self.codec_dtype, self._snac_dir())
        raise KeyError(node_name)

    # ---- request life cycle ----
    def get_sampling_config(self, model_kwargs):
        mk = dict(model_kwargs)
        mk.setdefault("temperature", 0.6)
        mk.setdefault("top_p", 0.8)
        mk.setdefault("repetition_penalty", 1.3)
        return super().get_sampling_config(mk)

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 4096))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, voice: str = "tara", **kw):
        text = f"{voice}: {prompt or ''}"
        tok = self._tokenizer()
        if tok is not None:
            ids = tok(text)["input_ids"]
        else:
            parts = (prompt or "").split()
            ids = [int(p) for p in parts] if parts and all(p.isdigit() for p in parts) else list(text.encode("utf-8"))
        ids = [128259] + [i % self.cfg.vocab_size for i in ids] + [128009, 128260]
        return {"input_ids": [torch.tensor(ids, dtype=torch.int64)]}

    def _snac_dir(self) -> str | None:
        """Where the codec's checkpoint is: ``snac_dir`` of the model kwargs, or a ``snac_24khz`` / ``snac`` directory
        beside the language model's files (the reference downloads ``hubertsiuzdak/snac_24khz`` separately)."""
        import os
        if self.skip_weight_loading:
            return None
        if self.snac_dir:
            return self.snac_dir
        for sub in ("snac_24khz", "snac"):
            d = os.path.join(self.model_dir or "", sub)
            if self.model_dir and os.path.exists(os.path.join(d, "pytorch_model.bin")):
                return d
        return None

    def _tokenizer(self):
        if self.model_dir is None:
            return None
        if not hasattr(self, "_tok"):
            try:
                from transformers import AutoTokenizer
                self._tok = AutoTokenizer.from_pretrained(self.model_dir)
            except Exception:  # noqa: BLE001
                self._tok = None
        return self._tok

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        if partition_name == "codec":
            return ForwardPassArgs({"graph_walk": "snac_chunk"}, [])
        return self.sm.initial(input_signals, self.get_max_output_tokens(model_kwargs))

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        if partition_name == "codec":
            return ForwardPassArgs(request_done=True)
        return self.sm.next(partition_metadata, persist_signals)

    def postprocess(self, output, modality, request_kwargs):
        if modality == "audio":
            return float_to_pcm16(output if isinstance(output, torch.Tensor) else torch.cat(list(output)))
        ids = output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output)
        return (" ".join(str(int(i)) for i in ids) + " ").encode()
