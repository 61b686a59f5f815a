"""Generic GQA transformer decoder over the paged KV pool, tensor-parallel aware.

One implementation serves the Llama-3.2 (Orpheus), Qwen2.5 (BAGEL und/gen experts), Qwen3 (Higgs, Qwen3-TTS
talker), Qwen3-MoE (Qwen3-Omni thinker/talker) and tiny test backbones; differences are configuration:
qkv bias, per-head QK-norm, rope flavour (plain / llama-3 scaled / multi-axis mRoPE), tied embeddings, MoE
layers, sliding window.

Per layer and step the kernels are: fused add+RMSNorm -> QKV GEMM (tcgen05) -> QK-norm+RoPE+KV-write ->
paged attention (tcgen05) -> o_proj GEMM [+ TP reduce] -> fused add+RMSNorm -> gate_up GEMM with SwiGLU
epilogue -> down GEMM [+ TP reduce]. Under tensor parallelism the row-parallel GEMMs hand their partial sums to
``tp_reduce`` (fused one-shot all-reduce over the symmetric heap, NCCL all-reduce as the baseline).

Reference counterparts: mstar/model/orpheus/components/language_model.py (115), mstar/model/components/
distributed/{linear,attention,mlp,embedding}.py, mstar/model/qwen3_omni/components/thinker.py:188-259.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
from torch import nn

from ..engine.cache_manager import BatchContext
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import _lib, gemm, norm as norm_ops, rope as rope_ops
from ..parallel.comm import CommGroup


@dataclass
class DecoderConfig:
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 688
    vocab_size: int = 32000
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_llama3: dict | None = None
    mrope_sections: list[int] | None = None
    mrope_interleaved: bool = True
    qkv_bias: bool = False
    qk_norm: bool = False
    tie_embeddings: bool = False
    sliding_window: int = 0
    has_lm_head: bool = True
    has_embedding: bool = True
    # MoE (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    moe_layers: list[int] | None = None      # None = all layers when num_experts > 0
    moe_expert_parallel: bool = False        # cut experts (not columns) over the tensor-parallel group
    dtype: torch.dtype = torch.bfloat16
    init_std: float = 0.02

    @property
    def n_pos_axes(self) -> int:
        return 3 if self.mrope_sections else 1


def _param(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, tp: CommGroup, bias: torch.Tensor | None = None,
                        partial_out: torch.Tensor | None = None):
    """y = all_reduce(x_shard @ w_shard.T): fused into the GEMM epilogue over the symmetric heap when attached.
    With ``partial_out`` (a slot of the symmetric heap) only this rank's partial product is written there and
    nothing is exchanged: the consumer kernel sums the ranks' slots (``TPFusedContext.reduce_norm``)."""
    if partial_out is not None:
        return gemm.linear(x, w, bias=bias if tp.rank == 0 else None, out=partial_out)
    if tp.size == 1:
        return gemm.linear(x, w, bias=bias)
    if tp.symm is not None and x.is_cuda:
        return tp.symm.linear_all_reduce(x, w, bias=bias)
    y = gemm.linear(x, w, bias=bias if tp.rank == 0 else None)
    return tp.all_reduce(y)


def tp_reduce(x: torch.Tensor, tp: CommGroup) -> torch.Tensor:
    """Sum row-parallel partials over the TP group (fused symmetric-heap path when attached)."""
    if tp.size == 1:
        return x
    if tp.symm is not None and x.is_cuda:
        return tp.symm.all_reduce(x)
    return tp.all_reduce(x)


# L2 management of the decode step (few token rows: every projection streams its weight once and is bound by its own
# latency chain, not by HBM). Each weight-streaming kernel asks the L2 for the weights of the kernel after it, so the
# HBM keeps working through the gaps, and marks what it streams itself evict-first. The amounts keep what is resident
# plus what is requested inside the 126 MB L2. Opt-in (MSTAR_L2_PREFETCH=1): on the 3B decode step at 64 requests it
# measured 4.19 ms against 4.14 ms without, i.e. no gain: the projections' fixed start and tail cost, not the weight
# stream, is what the step waits for.
L2_PREFETCH_MAX_ROWS = 256
L2_BUDGET = 96 << 20
L2_ATTN_PREFETCH = 64 << 20


def _l2_prefetch_on(h: torch.Tensor) -> bool:
    return (h.is_cuda and h.shape[0] <= L2_PREFETCH_MAX_ROWS and os.environ.get("MSTAR_L2_PREFETCH", "0") == "1")


def _wbytes(w) -> int:
    t = w.data
    return t.numel() * t.element_size()


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int, tp: CommGroup, device):
        super().__init__()
        self.cfg, self.layer_idx, self.tp = cfg, layer_idx, tp
        assert cfg.num_heads % tp.size == 0
        self.Hq = cfg.num_heads // tp.size
        self.Hkv = max(1, cfg.num_kv_heads // tp.size)
        self.D = cfg.head_dim
        H = cfg.hidden_size
        self.qkv_proj = _param(((self.Hq + 2 * self.Hkv) * self.D, H), cfg.dtype, device)
        self.qkv_bias = _param(((self.Hq + 2 * self.Hkv) * self.D,), cfg.dtype, device) if cfg.qkv_bias else None
        self.o_proj = _param((H, self.Hq * self.D), cfg.dtype, device)
        self.q_norm = _param((self.D,), cfg.dtype, device) if cfg.qk_norm else None
        self.k_norm = _param((self.D,), cfg.dtype, device) if cfg.qk_norm else None

    def forward(self, h: torch.Tensor, ctx: BatchContext, rope: "RopeTables",
                partial_out: torch.Tensor | None = None, next_w=None) -> torch.Tensor:
        """``next_w``: the weight of the projection that follows this block (the MLP's first), for the L2 requests."""
        pf = _l2_prefetch_on(h)
        if pf:
            _lib.prefetch_hint(self.o_proj)                     # fetched while the QKV projection runs
        qkv = gemm.linear(h, self.qkv_proj, bias=self.qkv_bias)
        kv = ctx.kv(self.layer_idx) if ctx.kv_layers else None
        q, _, _ = rope_ops.rope_kv(qkv, ctx.positions, rope.inv_freq, self.Hq, self.Hkv, self.D,
                                   axis_of_freq=rope.axis_of_freq, q_norm_w=self.q_norm, k_norm_w=self.k_norm,
                                   norm_eps=self.cfg.rms_eps, cache=kv, token_req=ctx.token_req,
                                   cache_pos=ctx.cache_pos, page_indptr=ctx.plan.page_indptr,
                                   page_indices=ctx.plan.page_indices)
        if pf and next_w is not None:
            _lib.prefetch_hint(next_w, 0, L2_ATTN_PREFETCH)     # while the K/V pages stream through, evict-first
        a = attn_ops.attention(q, ctx.plan, kv_cache=kv)
        if pf and next_w is not None:
            _lib.prefetch_hint(next_w, L2_ATTN_PREFETCH, max(0, L2_BUDGET - L2_ATTN_PREFETCH - _wbytes(self.o_proj)))
        elif pf:
            _lib.prefetch_hint(None, l2_hints=1)
        return row_parallel_linear(a.reshape(a.shape[0], self.Hq * self.D), self.o_proj, self.tp,
                                   partial_out=partial_out)


    def forward_folded(self, x: torch.Tensor, ctx: BatchContext, rope: "RopeTables", r: torch.Tensor,
                       norm_in, norm_out) -> None:
        """Attention block of a decode step with its norms folded into the projections: ``x`` is the QKV projection's
        input (the residual stream itself when ``norm_in`` carries its sums of squares), the output projection adds
        into the residual stream ``r`` in place and accumulates the stream's new sums of squares (``norm_out``)."""
        qkv = gemm.linear(x, self.qkv_proj, bias=self.qkv_bias, norm=norm_in)
        kv = ctx.kv(self.layer_idx) if ctx.kv_layers else None
        q, _, _ = rope_ops.rope_kv(qkv, ctx.positions, rope.inv_freq, self.Hq, self.Hkv, self.D,
                                   axis_of_freq=rope.axis_of_freq, q_norm_w=self.q_norm, k_norm_w=self.k_norm,
                                   norm_eps=self.cfg.rms_eps, cache=kv, token_req=ctx.token_req,
                                   cache_pos=ctx.cache_pos, page_indptr=ctx.plan.page_indptr,
                                   page_indices=ctx.plan.page_indices)
        a = attn_ops.attention(q, ctx.plan, kv_cache=kv)
        gemm.linear(a.reshape(a.shape[0], self.Hq * self.D), self.o_proj, residual=r, out=r, norm=norm_out)


class GatedMLP(nn.Module):
    """SwiGLU MLP; gate and up rows are stored interleaved so that the activation runs in the GEMM epilogue."""

    def __init__(self, hidden: int, inter: int, tp: CommGroup, dtype, device):
        super().__init__()
        self.tp = tp
        assert inter % tp.size == 0
        self.F = inter // tp.size
        self.gate_up_proj = _param((2 * self.F, hidden), dtype, device)
        self.down_proj = _param((hidden, self.F), dtype, device)

    def forward(self, h: torch.Tensor, reduce: bool = True, partial_out: torch.Tensor | None = None,
                next_w=None) -> torch.Tensor:
        """``next_w``: the weight that is streamed after this block (the next layer's QKV projection or the head)."""
        pf = _l2_prefetch_on(h)
        if pf:
            _lib.prefetch_hint(self.down_proj, 0, max(16 << 20, L2_BUDGET - _wbytes(self.gate_up_proj)))
        g = gemm.linear(h, self.gate_up_proj, epilogue=gemm.EPILOGUE_SWIGLU)
        if pf:
            if next_w is not None:
                _lib.prefetch_hint(next_w, 0, max(16 << 20, L2_BUDGET - _wbytes(self.down_proj)))
            else:
                _lib.prefetch_hint(None, l2_hints=1)
        if not reduce:
            return gemm.linear(g, self.down_proj)
        return row_parallel_linear(g, self.down_proj, self.tp, partial_out=partial_out)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int, tp: CommGroup, device):
        super().__init__()
        self.cfg = cfg
        self.input_layernorm = _param((cfg.hidden_size,), cfg.dtype, device)
        self.post_attention_layernorm = _param((cfg.hidden_size,), cfg.dtype, device)
        self.self_attn = Attention(cfg, layer_idx, tp, device)
        is_moe = cfg.num_experts > 0 and (cfg.moe_layers is None or layer_idx in cfg.moe_layers)
        if is_moe:
            from .moe import SparseMoeBlock
            self.mlp = SparseMoeBlock(cfg, tp, device)
        else:
            self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, tp, cfg.dtype, device)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None, ctx: BatchContext, rope, next_w=None) -> tuple:
        if residual is None:
            residual = x
            h, _ = norm_ops.norm(x, self.input_layernorm, self.cfg.rms_eps)
        else:
            h, residual = norm_ops.norm(x, self.input_layernorm, self.cfg.rms_eps, residual=residual)
        dense = isinstance(self.mlp, GatedMLP)
        a = self.self_attn(h, ctx, rope, next_w=self.mlp.gate_up_proj if dense else None)
        h, residual = norm_ops.norm(a, self.post_attention_layernorm, self.cfg.rms_eps, residual=residual)
        return (self.mlp(h, next_w=next_w) if dense else self.mlp(h)), residual

    def forward_tp_fused(self, h: torch.Tensor, residual: torch.Tensor, ctx: BatchContext, rope, tpf, site: int,
                         gamma_next: torch.Tensor, next_w=None):
        """Tensor-parallel layer without all-reduce kernels. ``h`` is the normalised input, ``residual`` the residual
        stream. Both row-parallel GEMMs write partial sums into heap slots; the two norm kernels of the layer (the
        post-attention norm and the NEXT layer's input norm, ``gamma_next``) sum them across ranks as they read."""
        M = h.shape[0]
        self.self_attn(h, ctx, rope, partial_out=tpf.partial_out(site, M), next_w=self.mlp.gate_up_proj)
        h, residual = tpf.reduce_norm(site, M, self.post_attention_layernorm, self.cfg.rms_eps, residual)
        self.mlp(h, partial_out=tpf.partial_out(site + 1, M), next_w=next_w)
        return tpf.reduce_norm(site + 1, M, gamma_next, self.cfg.rms_eps, residual)


class RopeTables:
    def __init__(self, cfg: DecoderConfig, device):
        self.inv_freq = rope_ops.make_inv_freq(cfg.head_dim, cfg.rope_theta, device, llama3=cfg.rope_llama3)
        self.axis_of_freq = None
        if cfg.mrope_sections:
            self.axis_of_freq = rope_ops.mrope_axis_table(cfg.mrope_sections, cfg.mrope_interleaved).to(device)


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig, tp: CommGroup | None = None, device="cpu", tp_max_tokens: int = 16384 + 256,
                 tp_max_logit_rows: int = 256):
        super().__init__()
        import os
        self.cfg = cfg
        self.tp = tp or CommGroup.trivial()
        self.device_ = torch.device(device)
        H, V = cfg.hidden_size, cfg.vocab_size
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, self.tp, device) for i in range(cfg.num_layers)])
        # Tensor-parallel fused path (GPU ranks with a symmetric heap, dense layers): row-parallel GEMMs leave partial
        # sums in heap slots that the following norm kernels reduce; embedding table and output head are cut by
        # vocabulary rows. MSTAR_TP_FUSED=0 keeps the all-reduce form (fused GEMM epilogue / NCCL) and full tables.
        self.tpf = None
        dense = all(isinstance(layer.mlp, GatedMLP) for layer in self.layers)
        if (self.tp.size > 1 and getattr(self.tp, "symm", None) is not None and self.device_.type == "cuda" and dense
                and cfg.dtype == torch.bfloat16 and H % 8 == 0 and os.environ.get("MSTAR_TP_FUSED", "1") != "0"):
            from ..parallel.tp_fused import TPFusedContext
            vp = cfg.has_embedding and cfg.has_lm_head and os.environ.get("MSTAR_TP_VOCAB_PARALLEL", "1") != "0"
            self.tpf = TPFusedContext(self.tp.symm, H, tp_max_tokens, vocab=V if vp else 0,
                                      max_logit_rows=tp_max_logit_rows if vp else 0)
        self.vocab_parallel = self.tpf is not None and self.tpf.vocab > 0
        if self.vocab_parallel:
            self.embed_tokens = nn.Parameter(self.tpf.alloc_table(), requires_grad=False)
        else:
            self.embed_tokens = _param((V, H), cfg.dtype, device) if cfg.has_embedding else None
        self.norm = _param((H,), cfg.dtype, device)
        self._head_packed = None
        self._packed = False
        self._norms_folded = False
        self.lm_head = None
        if cfg.has_lm_head and not cfg.tie_embeddings:
            self.lm_head = _param((self.tpf.rows_per_rank if self.vocab_parallel else V, H), cfg.dtype, device)
        self.rope = RopeTables(cfg, device)

    def vocab_rows(self, full: torch.Tensor) -> torch.Tensor:
        """The rows of a [vocab, hidden] checkpoint tensor that this rank keeps (all of them unless the vocabulary
        is cut over the tensor-parallel ranks)."""
        return self.tpf.shard_rows(full) if self.vocab_parallel else full

    # ---- weights ----
    @torch.no_grad()
    def init_random(self, seed: int = 0) -> "DecoderLM":
        """N(0, init_std) weights from a CPU generator, norms at one. Sharded ranks draw the full tensor and keep
        their slice, so TP ranks hold slices of the same model."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        cfg, tp = self.cfg, self.tp
        std = cfg.init_std

        def draw(shape):
            return torch.randn(shape, generator=g, dtype=torch.float32) * std

        if self.embed_tokens is not None:
            self.embed_tokens.copy_(self.vocab_rows(draw((cfg.vocab_size, cfg.hidden_size)).to(cfg.dtype)))
        Hq, Hkv, D, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_size
        for layer in self.layers:
            at = layer.self_attn
            q, k, v = draw((Hq * D, H)), draw((Hkv * D, H)), draw((Hkv * D, H))
            at.qkv_proj.copy_(shard_qkv(q, k, v, Hq, Hkv, D, tp.rank, tp.size).to(cfg.dtype))
            if at.qkv_bias is not None:
                at.qkv_bias.zero_()
            o = draw((H, Hq * D))
            at.o_proj.copy_(o[:, tp.rank * at.Hq * D:(tp.rank + 1) * at.Hq * D].to(cfg.dtype))
            if at.q_norm is not None:
                at.q_norm.fill_(1.0)
                at.k_norm.fill_(1.0)
            layer.input_layernorm.fill_(1.0)
            layer.post_attention_layernorm.fill_(1.0)
            if isinstance(layer.mlp, GatedMLP):
                F = cfg.intermediate_size
                gt, up, dn = draw((F, H)), draw((F, H)), draw((H, F))
                load_gated_mlp(layer.mlp, gt, up, dn, tp.rank, tp.size, cfg.dtype)
            else:
                layer.mlp.init_random(g, std)
        self.norm.fill_(1.0)
        if self.lm_head is not None:
            self.lm_head.copy_(self.vocab_rows(draw((cfg.vocab_size, cfg.hidden_size)).to(cfg.dtype)))
        if self.vocab_parallel:
            torch.cuda.synchronize(self.device_)
            self.tp.symm.barrier()          # every rank's table shard is in place before anyone gathers from it
            torch.cuda.synchronize(self.device_)
        return self

    def head_weight(self):
        if self._head_packed is not None:
            return self._head_packed
        return self.lm_head if self.lm_head is not None else self.embed_tokens

    @torch.no_grad()
    def quantize_moe_fp8(self) -> "DecoderLM":
        """Block-scaled e4m3 expert weights for every mixture-of-experts layer (after the weights are loaded)."""
        for layer in self.layers:
            if hasattr(layer.mlp, "quantize_fp8"):
                layer.mlp.quantize_fp8()
        return self

    @torch.no_grad()
    def pack_weights(self) -> "DecoderLM":
        """Re-store the projection weights tile by tile (``gemm.PackedWeight``) for the weight-streaming GEMMs of
        the decode step. CUDA only; call after the weights are loaded. A tied embedding keeps its plain table for
        the token gather and gets a packed copy for the output head."""
        if self.embed_tokens.device.type != "cuda" or self._packed:
            return self

        def repack(mod, name):
            w = getattr(mod, name)
            if isinstance(w, gemm.PackedWeight) or w is None or w.shape[1] % 8:
                return
            pw = gemm.pack_weight(w.data)
            delattr(mod, name)
            setattr(mod, name, pw)

        for layer in self.layers:
            repack(layer.self_attn, "qkv_proj")
            repack(layer.self_attn, "o_proj")
            if isinstance(layer.mlp, GatedMLP):
                repack(layer.mlp, "gate_up_proj")
                repack(layer.mlp, "down_proj")
        if self.cfg.has_lm_head:
            hw = self.lm_head if self.lm_head is not None else self.embed_tokens
            self._head_packed = gemm.pack_weight(hw.data)
            if self.lm_head is not None:
                del self.lm_head
                self.lm_head = None
        self._packed = True
        torch.cuda.empty_cache()
        return self

    @torch.no_grad()
    def fold_norms(self) -> "DecoderLM":
        """Fold every layer's RMSNorm gains into the projection that consumes the normalised stream (the input norm
        into the QKV weight, the post-attention norm into the gate / up weight; the gains become ones, so every
        other path computes the same function as before). Decode-sized batches then run WITHOUT norm kernels: each
        output / down projection adds the residual in its epilogue, writes the new residual stream and accumulates
        its per-token sum of squares, and the next projection multiplies its output rows by 1 / rms
        (``forward_hidden`` -> ``_forward_hidden_folded``). Dense layers, one tensor-parallel rank, plain (not yet
        packed) weights; call after the weights are loaded.

        Measured on the 3B decode step at 64 requests: 174 instead of 230 launches per step, but 4.01 ms against
        3.95 ms per step: replayed from a graph with dependent launch, the norm kernels already ran under their
        neighbours' start-up and the atomics lengthen the projections' tails. Models therefore call this only on
        request (``MSTAR_FOLD_NORMS=1``); the tiny test model always does, so that the GPU tests cover the path."""
        if self._norms_folded or self.tp.size > 1 or self._packed:
            return self
        if not all(isinstance(layer.mlp, GatedMLP) for layer in self.layers):
            return self
        for layer in self.layers:
            for w, g in ((layer.self_attn.qkv_proj, layer.input_layernorm),
                         (layer.mlp.gate_up_proj, layer.post_attention_layernorm)):
                w.data.copy_((w.data.float() * g.data.float()[None, :]).to(w.dtype))
                g.data.fill_(1.0)
        dev = self.norm.device
        self._ss = torch.zeros(2, 128, dtype=torch.float32, device=dev)      # per-token sums of squares: two streams
        self._norms_folded = True
        return self

    def _forward_hidden_folded(self, x: torch.Tensor, ctx: BatchContext) -> torch.Tensor:
        """Decode-sized forward with folded norms: 4 projections + RoPE + attention per layer, no norm kernels (one at
        the entry of the first layer, one before the head). The two accumulators alternate: each producer clears the
        one its successor will fill."""
        cfg = self.cfg
        H, eps = cfg.hidden_size, cfg.rms_eps
        r = x.reshape(-1, H)                                  # the residual stream, updated in place
        ss_a, ss_b = self._ss[0], self._ss[1]                 # after attention / after the MLP
        FN = gemm.FoldedNorm
        h0, _ = norm_ops.norm(r, self.layers[0].input_layernorm, eps)
        for i, layer in enumerate(self.layers):
            layer.self_attn.forward_folded(h0 if i == 0 else r, ctx, self.rope, r,
                                           None if i == 0 else FN(H, eps, ss_in=ss_b),
                                           FN(H, eps, ss_out=ss_a, ss_zero=ss_b))
            g = gemm.linear(r, layer.mlp.gate_up_proj, epilogue=gemm.EPILOGUE_SWIGLU, norm=FN(H, eps, ss_in=ss_a))
            gemm.linear(g, layer.mlp.down_proj, residual=r, out=r, norm=FN(H, eps, ss_out=ss_b, ss_zero=ss_a))
        h, _ = norm_ops.norm(r, self.norm, eps)
        return h

    # ---- forward ----
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self.vocab_parallel:
            return self.tpf.embed(input_ids.reshape(-1))
        return ew.embed(input_ids.reshape(-1), self.embed_tokens)

    def forward_hidden(self, x: torch.Tensor, ctx: BatchContext, deepstack=None) -> torch.Tensor:
        """x: [T, H] input embeddings -> final-normed hidden states [T, H]. ``deepstack`` = (int64 rows, [features
        [len(rows), H] per tapped encoder layer]): features k are added to the output of decoder layer k at those
        rows (the vision tower's intermediate taps of Qwen3-Omni / Qwen3-VL prompts)."""
        if deepstack is not None:
            rows, feats = deepstack
            residual = None
            for i, layer in enumerate(self.layers):
                x, residual = layer(x, residual, ctx, self.rope, next_w=self._weight_after(i))
                if i < len(feats):      # hidden = residual + x: adding to x adds to the hidden state
                    x = x.index_add(0, rows, feats[i].to(x.dtype))
            return norm_ops.norm(x, self.norm, self.cfg.rms_eps, residual=residual)[0]
        if self.tpf is not None and x.shape[0] <= self.tpf.max_tokens:
            x = x.reshape(-1, x.shape[-1])
            residual = self.tpf.residual_rows(x)
            h, _ = norm_ops.norm(x, self.layers[0].input_layernorm, self.cfg.rms_eps)
            n = len(self.layers)
            for i, layer in enumerate(self.layers):
                gamma_next = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
                h, residual = layer.forward_tp_fused(h, residual, ctx, self.rope, self.tpf, 2 * i, gamma_next,
                                                     next_w=self._weight_after(i))
            return h
        if self._norms_folded and x.shape[0] <= 128 and x.dtype == self.cfg.dtype:
            return self._forward_hidden_folded(x, ctx)
        residual = None
        for i, layer in enumerate(self.layers):
            x, residual = layer(x, residual, ctx, self.rope, next_w=self._weight_after(i))
        h, _ = norm_ops.norm(x, self.norm, self.cfg.rms_eps, residual=residual)
        return h

    def _weight_after(self, i: int):
        """The weight streamed after layer ``i``: the next layer's QKV projection, or the output head."""
        if i + 1 < len(self.layers):
            return self.layers[i + 1].self_attn.qkv_proj
        return self.head_weight() if self.cfg.has_lm_head else None

    def logits(self, hidden_rows: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
        if self.vocab_parallel and hidden_rows.shape[0] <= self.tpf.max_logit_rows:
            return self.tpf.logits(hidden_rows, self.head_weight())      # bf16, padded row pitch
        if self.vocab_parallel:
            raise ValueError(f"{hidden_rows.shape[0]} logit rows exceed the vocabulary-parallel logits buffer "
                             f"({self.tpf.max_logit_rows}): raise tp_max_logit_rows or set MSTAR_TP_VOCAB_PARALLEL=0")
        if _l2_prefetch_on(hidden_rows):
            _lib.prefetch_hint(None, l2_hints=1)      # the head's weight passes through the L2 once
        return gemm.linear(hidden_rows, self.head_weight(), out_dtype=out_dtype)

    def forward(self, ctx: BatchContext, input_ids: torch.Tensor | None = None,
                inputs_embeds: torch.Tensor | None = None, all_logits: bool = False,
                return_hidden: bool = False, deepstack=None):
        x = inputs_embeds if inputs_embeds is not None else self.embed(input_ids)
        h = self.forward_hidden(x, ctx, deepstack=deepstack)
        if return_hidden and not self.cfg.has_lm_head:
            return h
        rows = h if all_logits else h.index_select(0, ctx.logit_rows)
        lg = self.logits(rows)
        return (lg, h) if return_hidden else lg


def shard_qkv(q, k, v, Hq, Hkv, D, rank, size):
    """Rows of the fused QKV weight (or bias) held by one TP rank: its q heads, then its k heads, then v heads.
    KV heads are replicated when there are fewer of them than ranks."""
    hq = Hq // size
    qs = q[rank * hq * D:(rank + 1) * hq * D]
    if Hkv >= size:
        hk = Hkv // size
        ks, vs = k[rank * hk * D:(rank + 1) * hk * D], v[rank * hk * D:(rank + 1) * hk * D]
    else:
        rep = size // Hkv
        i = rank // rep
        ks, vs = k[i * D:(i + 1) * D], v[i * D:(i + 1) * D]
    return torch.cat([qs, ks, vs], dim=0)


@torch.no_grad()
def load_gated_mlp(mlp: GatedMLP, gate, up, down, rank, size, dtype):
    F = gate.shape[0] // size
    gs, us = gate[rank * F:(rank + 1) * F], up[rank * F:(rank + 1) * F]
    mlp.gate_up_proj.copy_(gemm.interleave_gate_up(gs, us).to(dtype))
    mlp.down_proj.copy_(down[:, rank * F:(rank + 1) * F].to(dtype))
