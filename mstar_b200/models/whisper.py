"""Whisper-large-v3 class speech recognition: log-mel -> encoder (stateless node) -> decoder with causal
self-attention over the paged KV pool and cross-attention to the encoder output.

The cross-attention keys / values of a request never change, so they are projected once at prefill into a static
pool (one slot per sampler slot, fixed stride per slot); the decode step reads them through a dense attention plan
whose offsets are computed on the device from the batch's slot ids, which keeps the step capturable in a CUDA graph.
The decoder has learned positions (no rotary embedding): the fused q/k/v kernel runs with zero frequencies, which
leaves q and k unrotated and still writes K/V into the pool's pages.

Reference counterparts: mstar/model/whisper/whisper_model.py (406 lines; CrossAttnKVConfig :95-112), submodules.py
(262), components/decoder.py (181; cross attention :78).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import GraphEdge, GraphNode
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from .base import small_scale, EngineType, Model
from .encoders import AudioEncoder, EncoderConfig, log_mel_spectrogram
from .llm_common import LMStateMachine, lm_walks
from .submodule_base import ARNodeSubmodule, BATCHED_LOGITS, NodeSubmodule

SOT, EOT, LANG_EN, TRANSCRIBE, TRANSLATE, NO_TS = 50258, 50257, 50259, 50360, 50359, 50364


def _p(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


class CrossAttnPool:
    """Static cross-attention K/V: [layers][slots * max_len, heads, D]; slot s owns rows [s*max_len, (s+1)*max_len)."""

    def __init__(self, layers, slots, max_len, heads, D, dtype, device):
        self.max_len, self.slots = max_len, slots
        self.k = torch.zeros((layers, slots * max_len, heads, D), dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.lens = torch.zeros(slots, dtype=torch.int32, device=device)

    def write(self, layer: int, slot: int, k: torch.Tensor, v: torch.Tensor) -> None:
        n = k.shape[0]
        self.k[layer, slot * self.max_len:slot * self.max_len + n] = k
        self.v[layer, slot * self.max_len:slot * self.max_len + n] = v
        self.lens[slot] = n

    def plan(self, q_indptr: torch.Tensor, row_slot: torch.Tensor, batch: int, n_tokens: int, n_tiles: int):
        """Dense plan over the pool for a batch whose entry b uses slot row_slot[b] (device arithmetic only)."""
        off = (row_slot.to(torch.int32) * self.max_len).to(torch.int32)
        kv_indptr = torch.cat([off, off[-1:] + self.max_len])
        return attn_ops.AttnPlan(q_indptr=q_indptr, kv_lens=self.lens[row_slot.long()].contiguous(), batch=batch,
                                 num_q_tokens=n_tokens, num_q_tiles=n_tiles, kv_indptr=kv_indptr.contiguous(),
                                 causal=False)


class WhisperDecoderLayer(nn.Module):
    def __init__(self, H, heads, ffn, dt, dev):
        super().__init__()
        self.ln1_w, self.ln1_b = _p((H,), dt, dev), _p((H,), dt, dev)
        self.qkv_w, self.qkv_b = _p((3 * H, H), dt, dev), _p((3 * H,), dt, dev)
        self.o_w, self.o_b = _p((H, H), dt, dev), _p((H,), dt, dev)
        self.ln2_w, self.ln2_b = _p((H,), dt, dev), _p((H,), dt, dev)
        self.cq_w, self.cq_b = _p((H, H), dt, dev), _p((H,), dt, dev)
        self.ckv_w, self.ckv_b = _p((2 * H, H), dt, dev), _p((2 * H,), dt, dev)
        self.co_w, self.co_b = _p((H, H), dt, dev), _p((H,), dt, dev)
        self.ln3_w, self.ln3_b = _p((H,), dt, dev), _p((H,), dt, dev)
        self.fc1_w, self.fc1_b = _p((ffn, H), dt, dev), _p((ffn,), dt, dev)
        self.fc2_w, self.fc2_b = _p((H, ffn), dt, dev), _p((H,), dt, dev)


class WhisperDecoder(nn.Module):
    def __init__(self, vocab=51866, hidden=1280, layers=32, heads=20, ffn=5120, max_pos=448, dtype=torch.bfloat16,
                 device="cpu"):
        super().__init__()
        self.H, self.heads, self.D, self.dtype, self.vocab = hidden, heads, hidden // heads, dtype, vocab
        self.tok = _p((vocab, hidden), dtype, device)
        self.pos = _p((max_pos, hidden), dtype, device)
        self.layers = nn.ModuleList([WhisperDecoderLayer(hidden, heads, ffn, dtype, device) for _ in range(layers)])
        self.lnf_w, self.lnf_b = _p((hidden,), dtype, device), _p((hidden,), dtype, device)
        self.zero_freq = torch.zeros(self.D // 2, dtype=torch.float32, device=device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if "ln" in n:
                p.data.fill_(1.0) if n.endswith("_w") else p.data.zero_()
            elif p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.dtype))
        return self

    def project_cross(self, feats: torch.Tensor, pool: CrossAttnPool, slot: int) -> None:
        for i, L in enumerate(self.layers):
            kv = gemm.linear(feats, L.ckv_w, bias=L.ckv_b)
            pool.write(i, slot, kv[:, :self.H].reshape(-1, self.heads, self.D),
                       kv[:, self.H:].reshape(-1, self.heads, self.D))

    def forward(self, ctx, ids: torch.Tensor, pool: CrossAttnPool) -> torch.Tensor:
        H, nh, D = self.H, self.heads, self.D
        pos = ctx.positions if ctx.positions.dim() == 1 else ctx.positions[0]
        x = ew.embed(ids.reshape(-1), self.tok) + self.pos[pos.long().clamp_max(self.pos.shape[0] - 1)]
        cplan = pool.plan(ctx.plan.q_indptr, ctx.row_slot, ctx.batch, ctx.num_tokens, ctx.plan.num_q_tiles)
        for i, L in enumerate(self.layers):
            h, _ = norm_ops.norm(x, L.ln1_w, 1e-5, bias=L.ln1_b, layernorm=True)
            qkv = gemm.linear(h, L.qkv_w, bias=L.qkv_b)
            kvc = ctx.kv(i)
            q, _, _ = rope_ops.rope_kv(qkv, pos, self.zero_freq, nh, nh, D, cache=kvc, token_req=ctx.token_req,
                                       cache_pos=ctx.cache_pos, page_indptr=ctx.plan.page_indptr,
                                       page_indices=ctx.plan.page_indices)
            a = attn_ops.attention(q, ctx.plan, kv_cache=kvc)
            x = gemm.linear(a.reshape(-1, H), L.o_w, bias=L.o_b, residual=x)
            h, _ = norm_ops.norm(x, L.ln2_w, 1e-5, bias=L.ln2_b, layernorm=True)
            q = gemm.linear(h, L.cq_w, bias=L.cq_b).reshape(-1, nh, D)
            a = attn_ops.attention(q, cplan, k=pool.k[i], v=pool.v[i])
            x = gemm.linear(a.reshape(-1, H), L.co_w, bias=L.co_b, residual=x)
            h, _ = norm_ops.norm(x, L.ln3_w, 1e-5, bias=L.ln3_b, layernorm=True)
            # the published weights were trained with the exact (erf) GELU; the GEMM's fused epilogue is the tanh form
            h = torch.nn.functional.gelu(gemm.linear(h, L.fc1_w, bias=L.fc1_b).float()).to(x.dtype)
            x = gemm.linear(h, L.fc2_w, bias=L.fc2_b, residual=x)
        h, _ = norm_ops.norm(x, self.lnf_w, 1e-5, bias=self.lnf_b, layernorm=True)
        rows = h.index_select(0, ctx.logit_rows)
        return gemm.linear(rows, self.tok, out_dtype=torch.float32)


class WhisperEncoderSubmodule(NodeSubmodule):
    def __init__(self, enc: AudioEncoder, device, n_mels: int, chunk_s: float = 30.0):
        super().__init__(device, enc.c.dtype)
        self.enc, self.n_mels, self.chunk = enc, n_mels, int(chunk_s * 16000)

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        wav = ni.tensor_inputs["audio"][0].float().reshape(-1)[:self.chunk]
        if wav.numel() < self.chunk and not ni.kwargs.get("no_pad"):
            wav = torch.nn.functional.pad(wav, (0, self.chunk - wav.numel()))
        mel = log_mel_spectrogram(wav.to(self.device), n_mels=self.n_mels)
        feats, _ = self.enc([mel])
        return {"audio_features": feats}


class WhisperDecoderSubmodule(ARNodeSubmodule):
    def __init__(self, dec: WhisperDecoder, device, pool_slots: int, max_audio_len: int, layers: int):
        super().__init__(device, dec.dtype)
        self.dec = dec
        self.pool = CrossAttnPool(layers, pool_slots, max_audio_len, dec.heads, dec.D, dec.dtype, device)

    def preprocess(self, graph_walk, engine_inputs, inputs):
        if graph_walk == "prefill":
            for ni in inputs:
                slot = engine_inputs.sampler.slot(ni.request_id)
                feats = ni.tensor_inputs["audio_features"][0].to(self.device, self.dec.dtype)[:self.pool.max_len]
                self.dec.project_cross(feats, self.pool, slot)
        return {}

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ids = torch.cat([ni.input_ids.reshape(-1) for ni in inputs]).to(self.device)
        return {BATCHED_LOGITS: self.dec(engine_inputs.batch_context, ids, self.pool)}

    def forward_graph(self, graph_walk, engine_inputs, static_ids, ctx):
        return {BATCHED_LOGITS: self.dec(ctx, static_ids, self.pool)}

    def can_use_cuda_graphs(self, graph_walk):
        return True

    def postprocess(self, request_id, request_info, outputs, inputs):
        tok = outputs["new_token"].to(torch.int64)
        return {"new_token": tok, "tok": tok, "last_token": tok}

    def check_stop(self, request_id, request_info, outputs):
        return {"decode_loop"} if outputs.get("new_token_host") == EOT else set()


class WhisperModel(Model):
    name = "whisper_large"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, max_batch: int = 32, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype, self.max_batch = small, dt, max_batch
        if small:
            k = small_scale()
            self.enc_cfg = EncoderConfig(64 * k, 2, 4, 16 * k, 128 * k, act="gelu_erf", dtype=dt, eps=1e-5)
            self.dec_kw = dict(vocab=51866, hidden=64 * k, layers=2, heads=4, ffn=128 * k)
            self.n_mels, self.max_audio = 16, 200
        else:
            self.enc_cfg = EncoderConfig(1280, 32, 20, 64, 5120, act="gelu_erf", dtype=dt, eps=1e-5)
            self.dec_kw = dict()
            self.n_mels, self.max_audio = 128, 1500
        self.sm = LMStateMachine("decoder")

    def get_graph_walk_graphs(self):
        enc = GraphNode("audio_encoder", {"audio"}, [GraphEdge("decoder", "audio_features")])
        return lm_walks("decoder", max_iters=448, prefill_inputs={"audio_features"}, pre_nodes=[enc])

    def get_node_engine_types(self):
        return {"audio_encoder": EngineType.STATELESS, "decoder": EngineType.KV_CACHE}

    def get_kv_cache_config(self):
        d = WhisperDecoder.__init__.__defaults__
        H, heads, layers = (64 * small_scale(), 4, 2) if self.small else (1280, 20, 32)
        return [KVCacheConfig(layers, heads, H // heads, max_seq_len=448, max_num_pages=16 if self.small else 256,
                              page_size=16 if self.small else 128, num_qo_heads=heads, nodes=["decoder"], dtype=self.dtype)]

    def get_engine_hints(self, node):
        return dict(vocab_size=51866, group=1, max_tokens=4096, track_seen=False, max_batch=self.max_batch)

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "audio_encoder":
            enc = AudioEncoder(self.enc_cfg, n_mels=self.n_mels, max_frames=self.max_audio, device=device)
            enc = self._load(enc, "encoder")
            return WhisperEncoderSubmodule(enc, device, self.n_mels, chunk_s=4.0 if self.small else 30.0)
        if node_name == "decoder":
            dec = self._load(WhisperDecoder(dtype=self.dtype, device=device, **self.dec_kw), "decoder")
            return WhisperDecoderSubmodule(dec, device, 2 * self.max_batch, self.max_audio, len(dec.layers))
        raise KeyError(node_name)

    def _load(self, module, half):
        """Random-init weights, or the Hugging Face checkpoint under ``model_dir`` (strict, original tensor names)."""
        if self.skip_weight_loading or self.model_dir is None:
            return module.init_random(0)
        from .checkpoints import load_whisper_decoder, load_whisper_encoder
        (load_whisper_encoder if half == "encoder" else load_whisper_decoder)(module, self.model_dir)
        return module

    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 440))

    def get_sampling_config(self, model_kwargs):
        mk = dict(model_kwargs)
        mk.setdefault("temperature", 0.0)
        return super().get_sampling_config(mk)

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, task: str = "transcribe", **kw):
        ids = [SOT, LANG_EN, TRANSLATE if task == "translate" else TRANSCRIBE, NO_TS]
        if not tensors.get("audio"):
            raise ValueError("speech recognition needs an audio input")
        return {"input_ids": [torch.tensor(ids, dtype=torch.int64)], "audio": [tensors["audio"][0].float()]}

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        return self.sm.initial(input_signals, self.get_max_output_tokens(model_kwargs),
                               [GraphEdge("audio_encoder", "audio", list(input_signals["audio"]))])

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        return self.sm.next(partition_metadata, persist_signals)

    def postprocess(self, output, modality, request_kwargs):
        ids = output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output)
        if self.tokenizer() is not None:          # the tokens' own bytes: a character split across tokens streams intact
            return self.decode_text([i for i in ids if i < SOT - 1])
        return (" ".join(str(int(i)) for i in ids) + " ").encode()
