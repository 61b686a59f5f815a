"""Speech-token generator ("talker"): an autoregressive decoder that emits the first codebook's code of every
audio frame, and a small code predictor that fills in the remaining codebooks of the frame.

Step structure (the same code runs eagerly and inside a captured CUDA graph): the predictor for frame t-1 runs at
the START of step t, from the hidden state and first code that step t-1 left in per-slot device buffers; its codes
are this step's ``codes`` output and, summed through the codebook embeddings (plus the conditioning row of the
step), the decoder's input. The decoder then produces the logits from which the engine samples frame t's first
code. Frames therefore leave one step late, and nothing in the step depends on host-side sampling results.

The predictor is a dense causal transformer over the short sequence [hidden, code_0 .. code_j]; sub-step j runs it
over j + 2 positions per request (all requests packed) and samples code j+1 from its own head.

Reference counterparts: Qwen3-Omni talker with CodePredictor "5 layers x 15 unrolled steps"
(mstar/model/qwen3_omni/components/talker.py, 549 lines), Qwen3-TTS talker
(mstar/model/qwen3_tts/components/talker.py, 316 lines).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import attention as attn_ops
from ..ops import gemm
from ..ops.sampling import SamplerState, SamplingConfig
from .decoder import DecoderConfig, DecoderLM, _param
from .dit import MoTGenTower
from .submodule_base import ARNodeSubmodule, BATCHED_LOGITS


class CodePredictor(nn.Module):
    def __init__(self, cfg: DecoderConfig, talker_hidden: int, n_sub: int, codebook: int, device="cpu"):
        super().__init__()
        self.cfg, self.n_sub, self.codebook = cfg, n_sub, codebook
        self.tower = MoTGenTower(cfg, device=device)          # run with a causal dense plan
        H = cfg.hidden_size
        self.in_proj = _param((H, talker_hidden), cfg.dtype, device)
        self.embed = _param((n_sub + 1, codebook, H), cfg.dtype, device)   # embeddings of codes 0 .. n_sub
        self.heads = _param((n_sub, codebook, H), cfg.dtype, device)
        self._plans: dict[tuple[int, int], tuple] = {}
        self.device = torch.device(device)

    def init_random(self, seed=0):
        self.tower.init_random(seed)
        g = torch.Generator().manual_seed(seed + 11)
        for p in (self.in_proj, self.embed, self.heads):
            p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1])).to(p.dtype))
        return self

    def _plan(self, B: int, L: int):
        key = (B, L)
        if key not in self._plans:
            G = self.cfg.num_heads // self.cfg.num_kv_heads
            plan = attn_ops.dense_plan([L] * B, [L] * B, G, self.device, causal=True)
            pos = torch.arange(L, dtype=torch.int32, device=self.device).repeat(B)
            last = torch.arange(B, device=self.device) * L + (L - 1)
            self._plans[key] = (plan, pos, last)
        return self._plans[key]

    def forward(self, hidden: torch.Tensor, code0: torch.Tensor, sampler: SamplerState | None, row_slot) -> torch.Tensor:
        """hidden [B, talker_hidden], code0 int64 [B] -> codes int64 [B, n_sub + 1] (code0 first)."""
        B = hidden.shape[0]
        H = self.cfg.hidden_size
        seq = torch.empty((B, self.n_sub + 2, H), dtype=self.cfg.dtype, device=hidden.device)
        seq[:, 0] = gemm.linear(hidden.to(self.cfg.dtype), self.in_proj)
        codes = [code0.clamp(0, self.codebook - 1)]
        seq[:, 1] = self.embed[0][codes[0]]
        for j in range(self.n_sub):
            L = j + 2
            plan, pos, last = self._plan(B, L)
            h = self.tower(seq[:, :L].reshape(B * L, H), pos, plan)
            logits = gemm.linear(h.index_select(0, last), self.heads[j], out_dtype=torch.float32)
            c = sampler.sample(logits, row_slot) if sampler is not None else logits.argmax(-1)
            codes.append(c)
            if j + 1 < self.n_sub:
                seq[:, L] = self.embed[j + 1][c]
        return torch.stack(codes, dim=1)

    def frame_embedding(self, codes: torch.Tensor, embed_dim_proj: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of the codebook embeddings of a frame: [B, H_predictor]."""
        e = self.embed[0][codes[:, 0]]
        for k in range(1, codes.shape[1]):
            e = e + self.embed[k][codes[:, k]]
        return e


class TalkerSubmodule(ARNodeSubmodule):
    """``cond_edge``: name of the per-step conditioning input (text ids for a TTS talker, upstream hidden states
    for an omni talker); ``cond_is_ids`` selects the embedding table vs. the projection."""

    def __init__(self, lm: DecoderLM, predictor: CodePredictor, device, *, num_slots: int, codec_eos: int,
                 cond_edge: str, cond_is_ids: bool, cond_dim: int, loop_name: str, frame_edge: str = "codec_frames",
                 text_vocab: int = 0, aux_cfg: SamplingConfig | None = None, suppress_from: int | None = None):
        super().__init__(device, lm.cfg.dtype)
        # ids from ``suppress_from`` up are the codec's control tokens: never sampled as a frame's first code, except
        # the end-of-speech id (reference: mstar/model/qwen3_omni/submodules.py:1290-1309)
        self.suppress = None
        if suppress_from is not None and suppress_from < lm.cfg.vocab_size:
            m = torch.zeros(lm.cfg.vocab_size, dtype=torch.bool, device=device)
            m[suppress_from:] = True
            if 0 <= codec_eos < lm.cfg.vocab_size:
                m[codec_eos] = False
            self.suppress = m
        self.lm, self.pred, self.codec_eos, self.loop_name, self.frame_edge = lm, predictor, codec_eos, loop_name, frame_edge
        self.cond_edge, self.cond_is_ids = cond_edge, cond_is_ids
        H, dt = lm.cfg.hidden_size, lm.cfg.dtype
        self.cond_table = _param((text_vocab, H), dt, device) if cond_is_ids else None
        self.cond_proj = None if cond_is_ids else _param((H, cond_dim), dt, device)
        self.frame_proj = _param((H, predictor.cfg.hidden_size), dt, device)
        self.pad_embed = _param((1, H), dt, device)
        self.bos_embed = _param((1, H), dt, device)
        g = torch.Generator().manual_seed(5)
        for p in (self.cond_table, self.cond_proj, self.frame_proj, self.pad_embed, self.bos_embed):
            if p is not None:
                p.data.copy_((torch.randn(p.shape, generator=g) * 0.02).to(dt))
        n_codes = predictor.n_sub + 1
        self.prev_hidden = torch.zeros((num_slots, H), dtype=dt, device=device)
        self.cond_next = torch.zeros((num_slots, H), dtype=dt, device=device)     # conditioning row of the next step
        self.aux = SamplerState(num_slots, predictor.codebook, device, track_seen=False)
        self.aux_cfg = aux_cfg or SamplingConfig(predictor.codebook, temperature=0.9, top_k=50)
        self.n_codes = n_codes

    def get_needed_cache_labels(self, graph_walk, fwd_info):
        return ["main"]

    def can_use_cuda_graphs(self, graph_walk):
        return "decode" in graph_walk

    def _cond_rows(self, ni) -> torch.Tensor | None:
        t = ni.tensor_inputs.get(self.cond_edge)
        if not t:
            return None
        if self.cond_is_ids:
            ids = torch.cat([x.reshape(-1) for x in t]).to(self.device).long().clamp(0, self.cond_table.shape[0] - 1)
            return self.cond_table[ids]
        h = torch.cat([x.reshape(-1, self.cond_proj.shape[1]) for x in t]).to(self.device, self.dtype)
        return gemm.linear(h, self.cond_proj)

    def prepare_inputs(self, graph_walk, fwd_info, inputs):
        ni = super().prepare_inputs(graph_walk, fwd_info, inputs)
        if "prefill" in graph_walk:
            t = inputs.get(self.cond_edge) or []
            n = sum(x.reshape(-1).numel() if self.cond_is_ids else x.reshape(-1, x.shape[-1]).shape[0] for x in t)
            ni.input_seq_len = n + 1                          # conditioning rows + the codec BOS row
            ni.input_ids = torch.zeros(ni.input_seq_len, dtype=torch.int64)
        return ni

    def preprocess(self, graph_walk, engine_inputs, inputs):
        for ni in inputs:
            slot = engine_inputs.sampler.slot(ni.request_id)
            if ni.request_id not in self.aux._slot_of:
                info = engine_inputs.per_request_info[ni.request_id]
                self.aux.assign(ni.request_id, self.aux_cfg, seed=(info.random_seed or 0) + 1, slot=slot)
            if "decode" in graph_walk:                        # this step's conditioning row (or padding)
                rows = self._cond_rows(ni)
                self.cond_next[slot] = rows[-1] if rows is not None and rows.shape[0] else self.pad_embed[0]
        return {}

    def cleanup_request(self, request_id):
        self.aux.release(request_id)

    def capture_state(self):
        return [self.prev_hidden, self.aux.offset]

    def _suppress(self, logits: torch.Tensor) -> torch.Tensor:
        """In place (a vocabulary-parallel head hands out a view of its own buffer, whose layout the sampler knows)."""
        if self.suppress is None:
            return logits
        n = min(self.suppress.numel(), logits.shape[-1])        # a head padded past the vocabulary keeps its pad columns
        if n != logits.shape[-1] or n != self.suppress.numel():
            logits[..., :n].masked_fill_(self.suppress[None, :n], -1e30)     # a view: nothing is allocated or cached
            return logits
        return logits.masked_fill_(self.suppress[None], -1e30)

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ctx = engine_inputs.batch_context
        if "prefill" in graph_walk:
            xs = []
            for ni in inputs:
                rows = self._cond_rows(ni)
                xs.append(self.bos_embed if rows is None else torch.cat([rows, self.bos_embed]))
            logits, hidden = self.lm(ctx, inputs_embeds=torch.cat(xs).contiguous(), return_hidden=True)
            self.prev_hidden[ctx.row_slot.long()] = hidden.index_select(0, ctx.logit_rows)
            return {BATCHED_LOGITS: self._suppress(logits)}
        ids = torch.cat([ni.input_ids.reshape(-1)[-1:] for ni in inputs]).to(self.device)
        return self._decode_step(ids, ctx)

    def forward_graph(self, graph_walk, engine_inputs, static_ids, ctx):
        return self._decode_step(static_ids, ctx)

    def _decode_step(self, code0: torch.Tensor, ctx):
        slots = ctx.row_slot.long()
        codes = self.pred(self.prev_hidden[slots], code0, self.aux, ctx.row_slot)          # frame t-1 complete
        x = gemm.linear(self.pred.frame_embedding(codes), self.frame_proj) + self.cond_next[slots]
        logits, hidden = self.lm(ctx, inputs_embeds=x.contiguous(), return_hidden=True)
        self.prev_hidden[slots] = hidden.index_select(0, ctx.logit_rows)
        return {BATCHED_LOGITS: self._suppress(logits), "codes": codes}

    def postprocess(self, request_id, request_info, outputs, inputs):
        tok = outputs["new_token"].to(torch.int64)
        out = {"tok": tok, "last_token": tok, "new_token": tok}
        if outputs.get("codes") is not None:
            out[self.frame_edge] = outputs["codes"].reshape(1, -1).to(torch.int64)
        return out

    def check_stop(self, request_id, request_info, outputs):
        sc = (request_info.sampling_config or {}).get("main", {})
        stop = not sc.get("ignore_eos", False) and outputs.get("new_token_host") == self.codec_eos
        return {self.loop_name} if stop else set()
