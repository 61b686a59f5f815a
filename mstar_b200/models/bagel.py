"""BAGEL-7B-MoT class unified understanding / generation model: one decoder with two sets of weights (a
"mixture of transformers": understanding expert for text and ViT tokens, generation expert for VAE latent tokens)
over a shared paged KV cache, a SigLIP-style NaViT encoder, a 2D latent autoencoder, and flow-matching image
generation with classifier-free guidance over up to three contexts (labels ``main`` = full context, ``cfg_text`` =
context without the text, ``cfg_img`` = context without the input image).

Two ways to run the guidance branches:
  * ``image_gen``: all branches packed into one forward of node ``LLM`` (one GPU);
  * ``image_gen_cfg``: CFG-parallel — nodes ``LLM``, ``LLM_cfg_text``, ``LLM_cfg_img`` on three GPUs run one branch
    each, ``combine_cfg`` merges the velocities, renormalises, takes the Euler step and feeds the latents back.

Prefill is ONE packed forward per context: every token carries an expert id, rows are split per expert for the
projections / norms / MLPs and joined for attention (``split_function_mot`` in the reference does the same per
layer).

Reference counterparts: mstar/model/bagel/bagel_model.py (walks :640-827), submodules.py (1570; gen step
:1005-1100, CFG combine :1478-1560), components/language_model.py (462; MoT split :58-84), vit_encoder.py (405),
autoencoder.py (322).
"""
from __future__ import annotations

import math

import torch

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop, Parallel, Sequential
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .decoder import DecoderConfig, DecoderLM, _param, row_parallel_linear
from .dit import MoTGenTower, sinusoidal_embedding
from .encoders import EncoderConfig, VisionEncoder
from .llm_common import lm_walks
from .schedulers import shifted_sigmas
from .submodule_base import ARNodeInputs, ARNodeSubmodule, BATCHED_LOGITS, NodeSubmodule
from .vae import ConvVAE, bagel_vae_config, tiny_vae_config
from .wan22 import VaeEncodeSubmodule

VISION_START, VISION_END, IMG_PLACEHOLDER, VAE_PLACEHOLDER, EOS = 151652, 151653, 151655, 151654, 151645
LABELS = ("main", "cfg_text", "cfg_img")


def bagel_7b_config(dtype) -> DecoderConfig:
    return DecoderConfig(hidden_size=3584, num_layers=28, num_heads=28, num_kv_heads=4, head_dim=128,
                         intermediate_size=18944, vocab_size=152064, rms_eps=1e-6, rope_theta=1e6, qkv_bias=True,
                         qk_norm=True, dtype=dtype)


def sincos_2d(h: int, w: int, dim: int, device) -> torch.Tensor:
    """Fixed 2D sine-cosine position table [h*w, dim] (half of the width per axis)."""
    q = dim // 4
    omega = 1.0 / (10000 ** (torch.arange(q, dtype=torch.float32, device=device) / q))
    ys, xs = torch.meshgrid(torch.arange(h, device=device), torch.arange(w, device=device), indexing="ij")
    parts = []
    for g in (xs, ys):
        a = g.reshape(-1, 1).float() * omega[None]
        parts += [torch.sin(a), torch.cos(a)]
    return torch.cat(parts, dim=1)


class BagelMoT(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, latent_dim: int, tp=None, device="cpu"):
        super().__init__()
        self.cfg, self.device = cfg, torch.device(device)
        self.und = DecoderLM(cfg, tp=tp, device=device)
        self.gen = MoTGenTower(cfg, tp=tp, device=device)
        H, dt = cfg.hidden_size, cfg.dtype
        self.vae2llm_w, self.vae2llm_b = _param((H, latent_dim), dt, device), _param((H,), dt, device)
        self.llm2vae_w, self.llm2vae_b = _param((latent_dim, H), dt, device), _param((latent_dim,), dt, device)
        self.t1_w, self.t1_b = _param((H, 256), dt, device), _param((H,), dt, device)
        self.t2_w, self.t2_b = _param((H, H), dt, device), _param((H,), dt, device)

    def init_random(self, seed=0):
        self.und.init_random(seed)
        self.gen.init_random(seed + 1)
        g = torch.Generator().manual_seed(seed + 2)
        for n, p in self.named_parameters():
            if not n.startswith(("und.", "gen.")):
                p.data.copy_((torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 1 else 1 / math.sqrt(p.shape[-1]))).to(p.dtype))
        return self

    def time_embed(self, t: torch.Tensor) -> torch.Tensor:
        e = gemm.linear(sinusoidal_embedding(t * 1000.0, 256).to(self.cfg.dtype), self.t1_w, bias=self.t1_b)
        return gemm.linear(torch.nn.functional.silu(e.float()).to(e.dtype), self.t2_w, bias=self.t2_b)

    def latent_tokens(self, lat_tok: torch.Tensor, grid: tuple[int, int], t: float) -> torch.Tensor:
        """[S, latent_dim] patch vectors -> embedded generation tokens (+ timestep, + 2D position)."""
        x = gemm.linear(lat_tok.to(self.cfg.dtype), self.vae2llm_w, bias=self.vae2llm_b)
        x = x + self.time_embed(torch.tensor([t], device=x.device))
        return x + sincos_2d(grid[0], grid[1], self.cfg.hidden_size, x.device).to(x.dtype)

    def forward_mixed(self, x: torch.Tensor, is_gen: torch.Tensor, ctx, spans=None) -> torch.Tensor:
        """Packed prefill with per-row experts. x: [T, H]; is_gen: bool [T]. K/V of every row go to the paged
        pool; returns final-normed hidden states [T, H] (understanding rows normed by the understanding expert).
        ``spans`` = (plan, rows) from ``BatchedCacheManager.span_plan``: those rows attend to everything up to the
        end of their span (an image's marker + patch rows see one another), every other row is causal — the same
        result as prefilling text, image, text as separate passes (mstar/model/bagel/submodules.py:378-380)."""
        cfg = self.cfg
        u_idx, g_idx = (~is_gen).nonzero().reshape(-1), is_gen.nonzero().reshape(-1)
        pos = ctx.positions if ctx.positions.dim() == 1 else ctx.positions[0]
        parts = {}
        for name, idx in (("u", u_idx), ("g", g_idx)):
            if idx.numel():
                parts[name] = dict(idx=idx, x=x.index_select(0, idx), res=None, pos=pos.index_select(0, idx).contiguous(),
                                   tr=ctx.token_req.index_select(0, idx).contiguous(),
                                   cp=ctx.cache_pos.index_select(0, idx).contiguous())
        T = x.shape[0]
        Hq = self.und.layers[0].self_attn.Hq
        for li in range(cfg.num_layers):
            kv = ctx.kv(li)
            q_full = torch.empty((T, Hq, cfg.head_dim), dtype=cfg.dtype, device=x.device)
            for name, p in parts.items():
                sub = dict(kv=kv, token_req=p["tr"], cache_pos=p["cp"], page_indptr=ctx.plan.page_indptr,
                           page_indices=ctx.plan.page_indices)
                if name == "g":
                    q, _, _, p["res"] = self.gen.layer_qkv(li, p["x"], p["res"], p["pos"], sub)
                else:
                    q, p["res"] = self._und_qkv(li, p["x"], p["res"], p["pos"], sub)
                q_full[p["idx"]] = q
            a = attn_ops.attention(q_full, ctx.plan, kv_cache=kv)
            if spans is not None:
                a.index_copy_(0, spans[1], attn_ops.attention(q_full.index_select(0, spans[1]), spans[0], kv_cache=kv))
            for name, p in parts.items():
                ai = a.index_select(0, p["idx"])
                if name == "g":
                    p["x"], p["res"] = self.gen.layer_out(li, ai, p["res"])
                else:
                    p["x"], p["res"] = self._und_out(li, ai, p["res"])
        out = torch.empty((T, cfg.hidden_size), dtype=cfg.dtype, device=x.device)
        for name, p in parts.items():
            w = self.gen.final_norm if name == "g" else self.und.norm
            out[p["idx"]] = norm_ops.norm(p["x"], w, cfg.rms_eps, residual=p["res"])[0]
        return out

    def _und_qkv(self, li, x, residual, pos, sub):
        layer, cfg = self.und.layers[li], self.cfg
        at = layer.self_attn
        if residual is None:
            residual = x.clone()
            h, _ = norm_ops.norm(x, layer.input_layernorm, cfg.rms_eps)
        else:
            h, residual = norm_ops.norm(x, layer.input_layernorm, cfg.rms_eps, residual=residual)
        qkv = gemm.linear(h, at.qkv_proj, bias=at.qkv_bias)
        q, _, _ = rope_ops.rope_kv(qkv, pos, self.und.rope.inv_freq, at.Hq, at.Hkv, at.D, q_norm_w=at.q_norm,
                                   k_norm_w=at.k_norm, norm_eps=cfg.rms_eps, cache=sub["kv"], token_req=sub["token_req"],
                                   cache_pos=sub["cache_pos"], page_indptr=sub["page_indptr"],
                                   page_indices=sub["page_indices"])
        return q, residual

    def _und_out(self, li, attn, residual):
        layer, cfg = self.und.layers[li], self.cfg
        at = layer.self_attn
        x = row_parallel_linear(attn.reshape(attn.shape[0], -1), at.o_proj, at.tp)
        h, residual = norm_ops.norm(x, layer.post_attention_layernorm, cfg.rms_eps, residual=residual)
        return layer.mlp(h), residual

    def gen_velocity(self, tokens: torch.Tensor, pos_id: list[int], n_branches: int, prefix_ctx) -> torch.Tensor:
        """tokens: [S, H] embedded noisy tokens; every branch b runs them at rotary position pos_id[b] against its
        cached context. Returns [n_branches, S, latent_dim] fp32."""
        S = tokens.shape[0]
        x = tokens.repeat(n_branches, 1)
        pos = torch.cat([torch.full((S,), p, dtype=torch.int32, device=tokens.device) for p in pos_id])
        G = max(1, self.gen.layers[0].Hq // self.gen.layers[0].Hkv)
        plan = attn_ops.dense_plan([S] * n_branches, [S] * n_branches, G, tokens.device, causal=False)
        h = self.gen(x, pos, plan, prefix_ctx=prefix_ctx)
        v = gemm.linear(h, self.llm2vae_w, bias=self.llm2vae_b, out_dtype=torch.float32)
        return v.reshape(n_branches, S, -1)


def image_span_positions(ids: list[int]):
    """Rotary positions of a packed prompt and its image spans. Text tokens advance the position by one; the rows
    from an image's start marker to its end marker share one position. Returns (int64 [T], [(start, end)] with
    ``end`` exclusive); an unterminated span runs to the end of the prompt."""
    pos, spans, p, open_at = [], [], 0, None
    for i, t in enumerate(ids):
        if i and (open_at is None or t == VISION_START):
            p += 1
        if t == VISION_START and open_at is None:
            open_at = i
        pos.append(p)
        if t == VISION_END and open_at is not None:
            spans.append((open_at, i + 1))
            open_at = None
    if open_at is not None:
        spans.append((open_at, len(ids)))
    return torch.tensor(pos, dtype=torch.int64), spans


def patchify2d(z: torch.Tensor, p: int = 2):
    """[C, H, W] -> ([h*w, p*p*C], (h, w)) with the channel fastest inside a patch."""
    C, H, W = z.shape
    h, w = H // p, W // p
    return z.reshape(C, h, p, w, p).permute(1, 3, 2, 4, 0).reshape(h * w, p * p * C).contiguous(), (h, w)


def unpatchify2d(tok: torch.Tensor, grid, C: int, p: int = 2):
    h, w = grid
    return tok.reshape(h, w, p, p, C).permute(4, 0, 2, 1, 3).reshape(C, h * p, w * p).contiguous()


def guidance_step(x, v: dict, dt: float, t: float, md: dict):
    """Guided velocity from the branch velocities, renormalised, and the Euler step. ``v``: label -> [S, D] fp32."""
    lo, hi = md.get("cfg_interval", (0.4, 1.0))
    s_text, s_img = float(md.get("cfg_text_scale", 4.0)), float(md.get("cfg_img_scale", 1.0))
    if not (lo < t <= hi) or "cfg_text" not in v:
        return x + dt * v["main"], v["main"]
    x_next, vv = ew.cfg_combine(v["main"].contiguous(), v["cfg_text"].contiguous(), x.contiguous(), dt, s_text,
                                v_img=v.get("cfg_img") if s_img != 1.0 else None, s_img=s_img,
                                renorm=md.get("cfg_renorm_type", "global") != "none",
                                renorm_min=float(md.get("cfg_renorm_min", 0.0)))
    return x_next, vv


class BagelLLMSubmodule(ARNodeSubmodule):
    """``branch`` = None: the node owns every label (packed guidance); else the one label this node serves."""

    def __init__(self, m: BagelMoT, device, latent_channels: int, num_steps: int, shift: float, branch: str | None = None):
        super().__init__(device, m.cfg.dtype)
        self.m, self.C, self.num_steps, self.shift, self.branch = m, latent_channels, num_steps, shift, branch

    def my_branch(self, kwargs: dict) -> str | None:
        """The single label this node serves, or None when it serves all (packed guidance on one GPU)."""
        return self.branch or ("main" if kwargs.get("cfg_parallel") else None)

    def my_labels(self, present: list[str], kwargs: dict) -> list[str]:
        b = self.my_branch(kwargs)
        return [lb for lb in present if b in (None, lb)]

    def get_needed_cache_labels(self, graph_walk, fwd_info):
        return list(LABELS) if self.branch is None else [self.branch]

    def can_use_cuda_graphs(self, graph_walk):
        return graph_walk == "decode"

    def max_batch_size(self, graph_walk):
        return 64 if graph_walk == "decode" else 1

    # ---- inputs ----
    def prepare_inputs(self, graph_walk, fwd_info, inputs):
        ni = ARNodeInputs(fwd_info.request_id, graph_walk, inputs, dict(fwd_info.step_metadata or {}))
        for key in ("input_ids", "tok"):
            if inputs.get(key):
                ni.input_ids = torch.cat([t.reshape(-1) for t in inputs[key]]).to(torch.int64).cpu()
                ni.input_seq_len = int(ni.input_ids.numel())
                break
        return ni

    @staticmethod
    def _context_rows(ids: torch.Tensor, label: str) -> torch.Tensor:
        """Rows of the packed prompt that belong to a label's context."""
        img = (ids == IMG_PLACEHOLDER) | (ids == VAE_PLACEHOLDER) | (ids == VISION_START) | (ids == VISION_END)
        if label == "cfg_text":
            return img.nonzero().reshape(-1)
        if label == "cfg_img":
            return (~img).nonzero().reshape(-1)
        return torch.arange(ids.numel())

    def custom_plan(self, cache, graph_walk, prepared):
        cfg = self.m.cfg
        G = max(1, cfg.num_heads // cfg.num_kv_heads)
        ni = prepared.node_inputs[0]
        if graph_walk.startswith("prefill"):
            labels = self.my_labels(list(ni.kwargs.get("labels", ["main"])), ni.kwargs)
            rows = {lb: self._context_rows(ni.input_ids, lb) for lb in labels}
            labels = [lb for lb in labels if rows[lb].numel()]
            ni.kwargs["_rows"], ni.kwargs["_labels"] = rows, labels
            # rotary position: text tokens advance by one; an image's start marker, patch rows and end marker share
            # one position (mstar/model/bagel/submodules.py:444-455, custom_advance_pos_id=1 at :833)
            ids = ni.input_ids
            pos_all, img_spans = image_span_positions(ids.tolist())
            ni.kwargs["_pos_end"] = int(pos_all[-1]) + 1 if ids.numel() else 0
            custom = torch.cat([pos_all[rows[lb]] for lb in labels]) if labels else None
            if not labels:
                labels, rows = ["main"], {"main": torch.zeros(0, dtype=torch.int64)}
            ctx = cache.plan([ni.request_id] * len(labels), [max(1, int(rows[lb].numel())) for lb in labels],
                             labels=labels, causal=True, group=G,
                             custom_positions=custom[None].to(torch.int32) if custom is not None else None)
            for lb in labels:
                cache.set_custom_pos_advance(ni.request_id, lb, int(ni.kwargs["_pos_end"]) - int(rows[lb].numel()))
            # rows of an image span attend among themselves: a second, non-causal pass over those rows
            spans = []
            for e, lb in enumerate(labels):
                where = {int(r): i for i, r in enumerate(rows[lb].tolist())}
                spans += [(e, where[a], where[b - 1] + 1) for a, b in img_spans if a in where and (b - 1) in where]
            ni.kwargs["_spans"] = cache.span_plan(ctx, spans, group=G) if spans else None
            return ctx
        if graph_walk == "decode":
            return None
        S = int(ni.kwargs["num_tokens"])
        labels = self.my_labels(list(ni.kwargs.get("branches", ["main"])), ni.kwargs)
        ni.kwargs["_labels"] = labels
        return cache.plan([ni.request_id] * len(labels), [S] * len(labels), labels=labels, causal=False,
                          write_cache=False, group=G)

    # ---- forwards ----
    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ctx, m = engine_inputs.batch_context, self.m
        ni = inputs[0]
        if graph_walk == "decode":
            ids = torch.cat([n.input_ids.reshape(-1)[-1:] for n in inputs]).to(self.device)
            return {BATCHED_LOGITS: m.und(ctx, input_ids=ids)}
        if graph_walk.startswith("prefill"):
            return [self._prefill(engine_inputs, ni, ctx)]
        return [self._gen_step(engine_inputs, ni, ctx)]

    def forward_graph(self, graph_walk, engine_inputs, static_ids, ctx):
        return {BATCHED_LOGITS: self.m.und(ctx, input_ids=static_ids)}

    def _prefill(self, ei, ni, ctx):
        m, ids = self.m, ni.input_ids.to(self.device)
        x = m.und.embed(ids)
        is_gen = ids == VAE_PLACEHOLDER
        feats = ni.tensor_inputs.get("image_features")
        if feats:
            f = torch.cat([t.reshape(-1, x.shape[-1]) for t in feats]).to(self.device, x.dtype)
            x[(ids == IMG_PLACEHOLDER).nonzero().reshape(-1)[:f.shape[0]]] = f
        lat = ni.tensor_inputs.get("image_latent")
        if lat:
            z = lat[0].to(self.device, torch.float32)
            tok, grid = patchify2d(z)
            x[is_gen.nonzero().reshape(-1)[:tok.shape[0]]] = m.latent_tokens(tok, grid, 0.0)
        rows, labels = ni.kwargs.pop("_rows"), ni.kwargs.pop("_labels")
        st = ei.per_request_states[ni.request_id]
        st["pos_end"] = ni.kwargs.pop("_pos_end")
        if not labels:
            return {"prefill_done": torch.zeros(1, dtype=torch.int64)}
        sel = torch.cat([rows[lb] for lb in labels]).to(self.device)
        h = m.forward_mixed(x.index_select(0, sel).contiguous(), is_gen.index_select(0, sel), ctx,
                            spans=ni.kwargs.pop("_spans", None))
        out = {"prefill_done": torch.tensor([ids.numel()], dtype=torch.int64)}
        if labels[0] == "main" and not ni.kwargs.get("gen"):          # first text token of an understanding request
            last = int(rows["main"].numel()) - 1
            out[BATCHED_LOGITS] = m.und.logits(h[last:last + 1])
        return out

    def _gen_step(self, ei, ni, ctx):
        st, md, m = ei.per_request_states[ni.request_id], ni.kwargs, self.m
        shape = tuple(md["latent_shape"])                        # [C, H, W]
        if ni.tensor_inputs.get("latents"):
            x = ni.tensor_inputs["latents"][-1].to(self.device, torch.float32)
        else:
            info = ei.per_request_info[ni.request_id]
            g = torch.Generator().manual_seed(int(md.get("seed", info.random_seed or 0)))
            x = patchify2d(torch.randn(shape, generator=g))[0].to(self.device)
        if st.get("gen_walk_id") != md.get("gen_id", 0):
            st["gen_walk_id"], st["step"] = md.get("gen_id", 0), 0
            st["sigmas"] = shifted_sigmas(int(md.get("num_steps", self.num_steps)), float(md.get("shift", self.shift)))
        i = st["step"]
        st["step"] += 1
        t, dt = st["sigmas"][i], st["sigmas"][i + 1] - st["sigmas"][i]
        grid = (shape[1] // 2, shape[2] // 2)
        labels = ni.kwargs.pop("_labels")
        tok = m.latent_tokens(x, grid, t)
        pos_end = st.get("pos_end", md.get("pos_end"))
        if pos_end is None:
            # the prompt passes ran in another pool (per-walk placement): the position after the prompt is what every
            # non-empty context of the request continues from
            alloc, pos_end = ei.cache_manager.alloc, 0
            for lb in alloc.get_labels(ni.request_id):
                s_ = alloc.get_state(ni.request_id, lb)
                pos_end = max(pos_end, s_.seq_len + s_.pos_offset if s_.seq_len else 0)
            st["pos_end"] = pos_end
        pos_end = int(pos_end)
        v = m.gen_velocity(tok, [pos_end] * len(labels), len(labels), ctx)
        vd = {lb: v[b] for b, lb in enumerate(labels)}
        branch = self.my_branch(md)
        if branch is not None:                                    # CFG-parallel: hand the branch velocity on
            return {"v_" + branch: vd[branch], "latents_echo": x}
        x_next, _ = guidance_step(x, vd, dt, t, md)
        return {"latents": x_next, "final_latents": unpatchify2d(x_next, grid, shape[0])}

    def postprocess(self, request_id, request_info, outputs, inputs):
        out = {k: v for k, v in outputs.items() if k not in ("new_token", "new_token_host")}
        if "new_token" in outputs and outputs["new_token"] is not None:
            tok = outputs["new_token"].to(torch.int64)
            out.update({"new_token": tok, "tok": tok, "last_token": tok})
        return out

    def check_stop(self, request_id, request_info, outputs):
        return {"decode_loop"} if outputs.get("new_token_host") == EOS else set()


class CombineCfgSubmodule(NodeSubmodule):
    """CFG-parallel merge: branch velocities from up to three GPUs -> guided velocity, renorm, Euler step."""

    def __init__(self, device, num_steps: int, shift: float):
        super().__init__(device, torch.float32)
        self.num_steps, self.shift = num_steps, shift

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        st, md = engine_inputs.per_request_states[ni.request_id], ni.kwargs
        if "sigmas" not in st:
            st["sigmas"] = shifted_sigmas(int(md.get("num_steps", self.num_steps)), float(md.get("shift", self.shift)))
            st["step"] = 0
        i = st["step"]
        st["step"] += 1
        t, dt = st["sigmas"][i], st["sigmas"][i + 1] - st["sigmas"][i]
        x = ni.tensor_inputs["latents_echo"][-1].to(self.device, torch.float32)
        v = {lb: ni.tensor_inputs["v_" + lb][-1].to(self.device, torch.float32) for lb in LABELS
             if ni.tensor_inputs.get("v_" + lb)}
        x_next, _ = guidance_step(x, v, dt, t, md)
        shape = tuple(md["latent_shape"])
        return {"latents": x_next, "final_latents": unpatchify2d(x_next, (shape[1] // 2, shape[2] // 2), shape[0])}


class VitSubmodule(NodeSubmodule):
    def __init__(self, enc: VisionEncoder, device):
        super().__init__(device, enc.c.dtype)
        self.enc = enc

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        feats, _, _ = self.enc([t.to(self.device) for t in ni.tensor_inputs["image"]])
        return {"image_features": feats}


class ImageDecodeSubmodule(NodeSubmodule):
    def __init__(self, vae: ConvVAE, device, dtype):
        super().__init__(device, dtype)
        self.vae = vae

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        z = ni.tensor_inputs["final_latents"][-1].to(self.device, self.dtype)
        return {"image": self.vae.decode(z[None])[0].float().cpu()}


class _BagelVaeEncode(VaeEncodeSubmodule):
    def forward(self, graph_walk, engine_inputs, ni, **kw):
        img = ni.tensor_inputs["image_vae"][0].to(self.device, self.dtype)
        return {"image_latent": self.vae.encode(img[None])[0].float()}


class BagelModel(Model):
    name = "bagel"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, num_steps: int | None = None,
                 max_num_pages: int | None = None, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        if small:
            k = small_scale()
            self.cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16 * k,
                                     intermediate_size=128 * k, vocab_size=152064, qkv_bias=True, qk_norm=True, dtype=dt)
            self.vae_cfg = tiny_vae_config(2, 4)
            self.vit_cfg, self.vit_patch = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, dtype=dt), 4
        else:
            self.cfg = bagel_7b_config(dt)
            self.vae_cfg = bagel_vae_config()
            self.vit_cfg, self.vit_patch = EncoderConfig(1152, 26, 16, 72, 4304, dtype=dt), 14
        self.num_steps = num_steps or (3 if small else 50)
        self.max_num_pages = max_num_pages or (64 if small else 1024)
        self.latent_dim = self.vae_cfg.latent_channels * 4

    # ---- structure ----
    def get_graph_walk_graphs(self):
        done = [GraphEdge(EMPTY_DESTINATION, "prefill_done", persist=True)]
        tok_outs = [GraphEdge(EMIT_TO_CLIENT, "new_token", output_modality="text", conductor_new_token=True),
                    GraphEdge(EMPTY_DESTINATION, "last_token", persist=True)]
        vit = GraphNode("vit_encoder", {"image"}, [GraphEdge("LLM", "image_features")])
        vae = GraphNode("vae_encoder", {"image_vae"}, [GraphEdge("LLM", "image_latent")])
        walks = {
            "prefill_text": GraphNode("LLM", {"input_ids"}, done + tok_outs),
            "prefill_vit": Sequential([vit, GraphNode("LLM", {"input_ids", "image_features"}, done + tok_outs)]),
            "prefill_vae": Sequential([Parallel([vit, vae]),
                                       GraphNode("LLM", {"input_ids", "image_features", "image_latent"}, done)]),
            "decode": lm_walks()["decode"],
        }
        dec = GraphNode("vae_decoder", {"final_latents"}, [GraphEdge(EMIT_TO_CLIENT, "image", output_modality="image")])
        step = GraphNode("LLM", {"latents"}, [GraphEdge("LLM", "latents"), GraphEdge(EMPTY_DESTINATION, "final_latents")],
                         enable_async_scheduling=False)
        walks["image_gen"] = Sequential([Loop(step, max_iters=self.num_steps, name="image_gen_loop",
                                              outputs=[GraphEdge("vae_decoder", "final_latents")]), dec])
        # CFG-parallel: three branch nodes, one combine node, latents fed back to all three
        names = {"main": "LLM", "cfg_text": "LLM_cfg_text", "cfg_img": "LLM_cfg_img"}
        branches = [GraphNode(n, {"latents"}, [GraphEdge("combine_cfg", "v_" + lb)] +
                              ([GraphEdge("combine_cfg", "latents_echo")] if lb == "main" else []),
                              enable_async_scheduling=False) for lb, n in names.items()]
        comb = GraphNode("combine_cfg", {"v_main", "v_cfg_text", "v_cfg_img", "latents_echo"},
                         [GraphEdge(n, "latents") for n in names.values()] + [GraphEdge(EMPTY_DESTINATION, "final_latents")],
                         enable_async_scheduling=False)
        walks["image_gen_cfg"] = Sequential([Loop(Sequential([Parallel(branches), comb]), max_iters=self.num_steps,
                                                  name="image_gen_loop",
                                                  outputs=[GraphEdge("vae_decoder", "final_latents")]), dec])
        walks["prefill_text_cfg"] = Parallel([GraphNode(n, {"input_ids"}, [GraphEdge(EMPTY_DESTINATION, "prefill_done_" + lb,
                                                                                   persist=True)])
                                              for lb, n in names.items()])
        return walks

    def get_optional_nodes(self):
        return {"LLM_cfg_text", "LLM_cfg_img", "combine_cfg"}       # only the guidance-parallel walks use them

    def get_node_engine_types(self):
        t = {n: EngineType.KV_CACHE for n in ("LLM", "LLM_cfg_text", "LLM_cfg_img")}
        t.update({n: EngineType.STATELESS for n in ("vit_encoder", "vae_encoder", "vae_decoder", "combine_cfg")})
        return t

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=32768, max_num_pages=self.max_num_pages,
                              page_size=16 if self.small else 128, num_qo_heads=c.num_heads, nodes=[n], dtype=c.dtype)
                for n in ("LLM", "LLM_cfg_text", "LLM_cfg_img")]

    def get_engine_hints(self, node):
        return dict(vocab_size=self.cfg.vocab_size, group=self.cfg.num_heads // self.cfg.num_kv_heads,
                    max_tokens=1 << 16, track_seen=False, max_batch=32)

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name.startswith("LLM"):
            m = BagelMoT(self.cfg, self.latent_dim, tp=tp_group, device=device)
            if self.skip_weight_loading or self.model_dir is None:
                m.init_random(0)
            else:
                # the published checkpoint: both experts, the latent / timestep projections (strict)
                import os
                from .checkpoints import load_bagel_mot
                ema = os.path.join(self.model_dir, "ema.safetensors")
                load_bagel_mot(m, ema if os.path.exists(ema) else self.model_dir)
            branch = {"LLM": None, "LLM_cfg_text": "cfg_text", "LLM_cfg_img": "cfg_img"}[node_name]
            sub = BagelLLMSubmodule(m, device, self.vae_cfg.latent_channels, self.num_steps, 3.0, branch)
            sub.node_name = node_name
            return sub
        if node_name == "vit_encoder":
            enc = VisionEncoder(self.vit_cfg, patch=self.vit_patch, pos="learned", pos_grid=8 if self.small else 70,
                                out_dim=self.cfg.hidden_size, device=device).init_random(0)
            if not (self.skip_weight_loading or self.model_dir is None):
                self._load_vit(enc)
            return VitSubmodule(enc, device)
        if node_name in ("vae_encoder", "vae_decoder"):
            vae = ConvVAE(self.vae_cfg)
            if not (self.skip_weight_loading or self.model_dir is None):
                import os
                from .checkpoints import load_image_autoencoder
                load_image_autoencoder(vae, os.path.join(self.model_dir, "ae.safetensors"))
            vae = vae.to(device=device, dtype=self.dtype).eval()
            if node_name == "vae_decoder":
                return ImageDecodeSubmodule(vae, device, self.dtype)
            return _BagelVaeEncode(vae, device, self.dtype)
        if node_name == "combine_cfg":
            return CombineCfgSubmodule(device, self.num_steps, 3.0)
        raise KeyError(node_name)

    def _load_vit(self, enc) -> None:
        """Vision tower + connector of the published checkpoint: SigLIP names under ``vit_model.``, the two-layer
        connector under ``connector.`` (this encoder's output projector), the learned position table under
        ``vit_pos_embed.pos_embed``."""
        import os
        from .checkpoints import CheckpointMismatch, iter_checkpoint, load_siglip_vision
        ema = os.path.join(self.model_dir, "ema.safetensors")
        tensors = {k: v for k, v in iter_checkpoint(ema if os.path.exists(ema) else self.model_dir)
                   if k.startswith(("vit_model.", "connector.", "vit_pos_embed."))}
        side = {"connector.fc1.weight": enc.proj1_w, "connector.fc1.bias": enc.proj1_b,
                "connector.fc2.weight": enc.proj2_w, "connector.fc2.bias": enc.proj2_b,
                "vit_pos_embed.pos_embed": enc.pos_table}
        for k, p in side.items():
            t = tensors.pop(k, None)
            if t is None or tuple(t.shape) != tuple(p.shape):
                raise CheckpointMismatch(f"BAGEL vision tower: {k} missing or of shape {None if t is None else tuple(t.shape)}"
                                         f" (parameter {tuple(p.shape)})")
            p.data.copy_(t.to(p.dtype))
        vit = {k[len("vit_model."):]: v for k, v in tensors.items() if k.startswith("vit_model.")}
        load_siglip_vision(enc, vit, position_table=False)

    # ---- request life cycle ----
    def get_max_output_tokens(self, model_kwargs=None):
        return int((model_kwargs or {}).get("max_tokens", 1024))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        v = self.cfg.vocab_size
        text = self.encode_text(prompt if "image" in (output_modalities or []) else self.chat_text(prompt), v, 1000)
        ids, out = [], {}
        gen = "image" in (output_modalities or [])
        if tensors.get("image"):
            im = tensors["image"][0].float()
            p = self.vit_patch
            n_vit = (im.shape[-2] // p) * (im.shape[-1] // p)
            ids += [VISION_START] + [IMG_PLACEHOLDER] * n_vit + [VISION_END]
            out["image"] = [im]
            if gen:       # editing: the input image also enters as clean latents of the generation expert
                sf = self.vae_cfg.spatial_factor
                n_vae = (im.shape[-2] // sf // 2) * (im.shape[-1] // sf // 2)
                ids += [VISION_START] + [VAE_PLACEHOLDER] * n_vae + [VISION_END]
                out["image_vae"] = [im * 2 - 1 if im.min() >= 0 else im]
        ids += text
        out["input_ids"] = [torch.tensor([i % v for i in ids] or [0], dtype=torch.int64)]
        return out

    def latent_shape(self, mk: dict) -> list[int]:
        sf = self.vae_cfg.spatial_factor
        H, W = int(mk.get("height", 16 if self.small else 1024)), int(mk.get("width", 16 if self.small else 1024))
        return [self.vae_cfg.latent_channels, H // sf, W // sf]

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        gen = "image" in (output_modalities or [])
        mk = model_kwargs or {}
        edges = [GraphEdge("LLM", "input_ids", list(input_signals["input_ids"]))]
        labels = ["main"]
        if gen:
            labels = ["main", "cfg_text"] + (["cfg_img"] if input_signals.get("image") and float(mk.get("cfg_img_scale", 1.0)) != 1.0 else [])
        if input_signals.get("image_vae"):
            walk = "prefill_vae"
            edges += [GraphEdge("vit_encoder", "image", list(input_signals["image"])),
                      GraphEdge("vae_encoder", "image_vae", list(input_signals["image_vae"]))]
        elif input_signals.get("image"):
            walk = "prefill_vit"
            edges.append(GraphEdge("vit_encoder", "image", list(input_signals["image"])))
        elif gen and mk.get("cfg_parallel"):
            walk = "prefill_text_cfg"
            edges += [GraphEdge(n, "input_ids", list(input_signals["input_ids"])) for n in ("LLM_cfg_text", "LLM_cfg_img")]
        else:
            walk = "prefill_text"
        return ForwardPassArgs({"graph_walk": walk, "max_tokens": self.get_max_output_tokens(mk)}, edges,
                               step_metadata={"labels": labels, "cfg_parallel": walk == "prefill_text_cfg", "gen": gen})

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        mk = md.get("model_kwargs") or {}
        fw = md["finished_walk"]
        gen = "image" in (md.get("output_modalities") or [])
        if fw.startswith("prefill") and gen:
            shape = self.latent_shape(mk)
            steps = int(mk.get("num_steps", self.num_steps))
            cfgp = fw == "prefill_text_cfg"
            branches = ["main", "cfg_text"] + (["cfg_img"] if cfgp or float(mk.get("cfg_img_scale", 1.0)) != 1.0 else [])
            step_md = {k: mk[k] for k in ("cfg_text_scale", "cfg_img_scale", "cfg_interval", "cfg_renorm_type",
                                          "cfg_renorm_min", "shift", "seed") if k in mk}
            step_md.update(num_steps=steps, latent_shape=shape, num_tokens=(shape[1] // 2) * (shape[2] // 2),
                           branches=branches, cfg_parallel=cfgp)
            nodes = ("LLM", "LLM_cfg_text", "LLM_cfg_img") if cfgp else ("LLM",)
            return ForwardPassArgs({"graph_walk": "image_gen_cfg" if cfgp else "image_gen",
                                    "dynamic_loop_iter_counts": {"image_gen_loop": steps}},
                                   [GraphEdge(n, "latents", []) for n in nodes], step_metadata=step_md)
        budget = md["max_tokens"] - md["tokens_out"]
        if fw.startswith("prefill") and budget > 0 and persist_signals.get("last_token"):
            last = persist_signals.pop("last_token")
            return ForwardPassArgs({"graph_walk": "decode", "max_tokens": budget,
                                    "dynamic_loop_iter_counts": {"decode_loop": budget}},
                                   [GraphEdge("LLM", "tok", last[-1:])], unpersist_tensors=[t.uuid for t in last])
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        if modality == "image":
            from ..api_server.media_io import tensor_to_png
            return tensor_to_png(output if isinstance(output, torch.Tensor) else output[-1])
        return self.decode_text(output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output))
