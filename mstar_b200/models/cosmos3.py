"""Cosmos3-class world model: one dual-pathway transformer node ``dit`` — a causal understanding tower whose K/V
for the prompt (label ``main``) and the negative prompt (label ``uncond``) are written to the paged pool by the
``prefill`` walks, and a generation tower that denoises latent video / image tokens against those cached prefixes
— plus a causal 3D VAE and an audio decoder. Both guidance branches of a step run as one packed forward.

Parallelism: the generation tower shards heads / FFN over the tensor-parallel group and the token rows over the
sequence-parallel group (Ulysses exchange around attention); the understanding tower is cut tp*sp ways over the
whole instance so that the prefix K/V a rank caches are exactly the heads it attends with after the exchange.

Walks: ``prefill`` (text), ``prefill_cond`` (text + conditioning image -> clean first-frame latent), ``image_gen``,
``video_gen``, ``video_sound_gen`` (+ ``audio_decoder``), ``action_gen`` (robot action chunk denoised as a short
token sequence). Denoise loops get their iteration count per request.

Reference counterparts: mstar/model/cosmos3/cosmos3_model.py (walks :220-454, sharding :209-218), submodules.py
(preprocess / plan :663-796, _forward_image_gen :872-919, captured variant :1507-1575), components/transformer.py,
packing.py, sound_tokenizer.py, config.py (:88-97 shape, :167-172 graph limits).
"""
from __future__ import annotations

import math

import torch

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop, Parallel, Sequential
from ..ops import attention as attn_ops
from ..ops import gemm
from ..parallel.comm import CommGroup
from ..parallel.sequence_parallel import gather_sequence, sp_seq_split
from .base import small_scale, EngineType, ForwardPassArgs, Model, seeded_init
from .sound_decoder import SoundDecoder, load_sound_decoder, pcm_layout, sound_decoder_config
from .decoder import DecoderConfig, DecoderLM, _param
from .dit import MoTGenTower, grid_positions, patchify, sinusoidal_embedding, unpatchify
from .schedulers import FlowUniPC
from .submodule_base import ARNodeInputs, ARNodeSubmodule, NodeSubmodule
from .vae import ConvVAE, cosmos3_vae_config, tiny_vae_config
from .wan22 import VaeDecodeSubmodule, VaeEncodeSubmodule


def cosmos3_nano_config(dtype=torch.bfloat16) -> DecoderConfig:
    return DecoderConfig(hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128,
                         intermediate_size=12288, vocab_size=151936, rms_eps=1e-6, rope_theta=1e6, qk_norm=True,
                         mrope_sections=[24, 20, 20], has_lm_head=False, dtype=dtype)


class Cosmos3Transformer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, latent_channels: int, patch=(1, 2, 2), action_dim: int = 32,
                 tp: CommGroup | None = None, sp: CommGroup | None = None, device="cpu", sound_dim: int = 64,
                 num_domains: int = 32):
        super().__init__()
        tp, sp = tp or CommGroup.trivial(), sp or CommGroup.trivial()
        inst = tp.instance or sp.instance or (tp if sp.size == 1 else sp)
        self.cfg, self.tp, self.sp, self.patch, self.C = cfg, tp, sp, patch, latent_channels
        self.und = DecoderLM(cfg, tp=inst, device=device)
        self.gen = MoTGenTower(cfg, tp=tp, sp=sp, device=device)
        H, dt = cfg.hidden_size, cfg.dtype
        pd = latent_channels * math.prod(patch)
        self.proj_in_w, self.proj_in_b = _param((H, pd), dt, device), _param((H,), dt, device)
        self.proj_out_w, self.proj_out_b = _param((pd, H), dt, device), _param((pd,), dt, device)
        self.t1_w, self.t1_b = _param((H, 256), dt, device), _param((H,), dt, device)
        self.t2_w, self.t2_b = _param((H, H), dt, device), _param((H,), dt, device)
        # robot actions: one full (weight, bias) pair per embodiment domain, stored as rows of two tables (the
        # published layout: row d of ``fc`` is that domain's [in, out] matrix, flattened)
        self.action_dim, self.num_domains = action_dim, num_domains
        self.act_in_fc, self.act_in_bias = _param((num_domains, action_dim * H), dt, device), _param((num_domains, H), dt, device)
        self.act_out_fc = _param((num_domains, H * action_dim), dt, device)
        self.act_out_bias = _param((num_domains, action_dim), dt, device)
        self.action_modality_embed = _param((H,), dt, device)
        self.audio_modality_embed = _param((H,), dt, device)
        self._domain_w: dict = {}
        # sound latents ([sound_dim] per latent frame) enter and leave the generation tower through their own pair
        # of projections and are denoised jointly with the video tokens
        self.sound_dim = sound_dim
        self.audio_in_w, self.audio_in_b = _param((H, sound_dim), dt, device), _param((H,), dt, device)
        self.audio_out_w, self.audio_out_b = _param((sound_dim, H), dt, device), _param((sound_dim,), dt, device)
        self.device = torch.device(device)

    def init_random(self, seed=0):
        self.und.init_random(seed)
        self.gen.init_random(seed + 1)
        g = torch.Generator().manual_seed(seed + 2)
        for n, p in self.named_parameters():
            if n.startswith(("und.", "gen.")):
                continue
            p.data.copy_((torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 1 else 1 / math.sqrt(p.shape[-1]))).to(p.dtype))
        return self

    def action_weights(self, domain: int):
        """(in weight [H, A], in bias [H], out weight [A, H], out bias [A]) of one embodiment domain, in the
        [out, in] orientation the GEMM takes; built once per domain."""
        w = self._domain_w.get(domain)
        if w is None:
            H, A = self.cfg.hidden_size, self.action_dim
            w = (self.act_in_fc[domain].view(A, H).t().contiguous(), self.act_in_bias[domain].contiguous(),
                 self.act_out_fc[domain].view(H, A).t().contiguous(), self.act_out_bias[domain].contiguous())
            self._domain_w[domain] = w
        return w

    def time_embed(self, t: torch.Tensor) -> torch.Tensor:
        e = sinusoidal_embedding(t, 256).to(self.cfg.dtype)
        e = gemm.linear(e, self.t1_w, bias=self.t1_b)
        return gemm.linear(torch.nn.functional.silu(e.float()).to(e.dtype), self.t2_w, bias=self.t2_b)

    def denoise(self, tokens: torch.Tensor, positions: torch.Tensor, t: float, n_branches: int, prefix_ctx,
                out_w=None, out_b=None) -> torch.Tensor:
        """tokens: [S, H] embedded noisy tokens of ONE request; runs ``n_branches`` guidance branches packed as
        [branch0 | branch1 | ...] and returns [n_branches, S, out] fp32 (``out_w=None``: the hidden states
        [n_branches, S, H], for callers that project bands of the sequence with different heads)."""
        S = tokens.shape[0]
        x = tokens + self.time_embed(torch.tensor([t], device=tokens.device))
        x = x.repeat(n_branches, 1)
        pos = positions.repeat(1, n_branches)
        S_tot = S * n_branches
        Hq_l = self.gen.layers[0].Hq // self.sp.size
        G = max(1, Hq_l // max(1, self.gen.layers[0].Hkv // self.sp.size))
        plan = attn_ops.dense_plan([S] * n_branches, [S] * n_branches, G, tokens.device, causal=False)
        if self.sp.size > 1:
            off = sp_seq_split(S_tot, self.sp.size)
            lo, hi = off[self.sp.rank], off[self.sp.rank + 1]
            h = self.gen(x[lo:hi].contiguous(), pos[:, lo:hi].contiguous(), plan, prefix_ctx=prefix_ctx, S_total=S_tot)
            if out_w is not None:
                # the output head runs on this rank's rows and only ITS result is gathered: [S, patch dim] fp32
                # instead of [S, hidden] bf16 (a 32 x smaller exchange at hidden 4096 and a 64-wide patch)
                out = gemm.linear(h, out_w, bias=out_b, out_dtype=torch.float32)
                return gather_sequence(out, self.sp, S_tot).reshape(n_branches, S, -1)
            h = gather_sequence(h, self.sp, S_tot)
        else:
            h = self.gen(x, pos, plan, prefix_ctx=prefix_ctx, S_total=S_tot)
        if out_w is None:
            return h.reshape(n_branches, S, -1)
        out = gemm.linear(h, out_w, bias=out_b, out_dtype=torch.float32)
        return out.reshape(n_branches, S, -1)


class Cosmos3DiTSubmodule(ARNodeSubmodule):
    LABELS = ("main", "uncond")

    def __init__(self, model: Cosmos3Transformer, device, default_steps: int, shift: float):
        super().__init__(device, model.cfg.dtype)
        self.m, self.default_steps, self.shift = model, default_steps, shift

    def get_needed_cache_labels(self, graph_walk, fwd_info):
        return list(self.LABELS)

    def can_batch(self, graph_walk):
        return graph_walk.startswith("prefill")

    def max_batch_size(self, graph_walk):
        return 8 if graph_walk.startswith("prefill") else 1

    def prepare_inputs(self, graph_walk, fwd_info, inputs):
        ni = ARNodeInputs(fwd_info.request_id, graph_walk, inputs, dict(fwd_info.step_metadata or {}))
        if graph_walk.startswith("prefill"):
            ni.input_ids = torch.cat([t.reshape(-1) for t in inputs.get("input_ids", [])]).to(torch.int64)
            ni.input_seq_len = int(ni.input_ids.numel())
        return ni

    # ---- planning: several (request, label) entries per request ----
    def custom_plan(self, cache, graph_walk, prepared):
        G = max(1, self.m.cfg.num_heads // self.m.cfg.num_kv_heads)
        if graph_walk.startswith("prefill"):
            rids, labels, qls = [], [], []
            for ni in prepared.node_inputs:
                neg = torch.cat([t.reshape(-1) for t in ni.tensor_inputs.get("neg_input_ids", [])] or [torch.zeros(0)])
                ni.kwargs["_neg_ids"] = neg.to(torch.int64)
                rids += [ni.request_id, ni.request_id]
                labels += ["main", "uncond"]
                qls += [ni.input_seq_len, max(1, int(neg.numel()))]
            return cache.plan(rids, qls, labels=labels, causal=True, group=G)
        ni = prepared.node_inputs[0]
        S = int(ni.kwargs["num_tokens"])
        nb = 2 if float(ni.kwargs.get("guidance_scale", 1.0)) != 1.0 else 1
        return cache.plan([ni.request_id] * nb, [S] * nb, labels=list(self.LABELS[:nb]), causal=False,
                          write_cache=False, group=G)

    # ---- forwards ----
    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ctx = engine_inputs.batch_context
        if graph_walk.startswith("prefill"):
            ids = []
            for ni in inputs:
                neg = ni.kwargs.pop("_neg_ids")
                ids += [ni.input_ids, neg if neg.numel() else torch.zeros(1, dtype=torch.int64)]
            x = self.m.und.embed(torch.cat(ids).to(self.device))
            self.m.und.forward_hidden(x, ctx)
            outs = []
            for ni in inputs:
                st = engine_inputs.per_request_states[ni.request_id]
                st["text_len"] = ni.input_seq_len
                o = {"prefill_done": torch.tensor([ni.input_seq_len], dtype=torch.int64)}
                if ni.tensor_inputs.get("image_latent"):
                    st["cond_latent"] = ni.tensor_inputs["image_latent"][0].to(self.device, torch.float32)
                outs.append(o)
            return outs
        return [self._gen_step(graph_walk, engine_inputs, inputs[0], ctx)]

    def _gen_step(self, walk, ei, ni, ctx):
        st, md = ei.per_request_states[ni.request_id], ni.kwargs
        m = self.m
        action = walk == "action_gen"
        if ni.tensor_inputs.get("latents"):
            x = ni.tensor_inputs["latents"][-1].to(self.device, torch.float32)
        else:
            info = ei.per_request_info[ni.request_id]
            g = torch.Generator().manual_seed(int(md.get("seed", info.random_seed or 0)))
            x = torch.randn(tuple(md["latent_shape"]), generator=g).to(self.device)
        if "sched" not in st or st.get("sched_walk") != walk:
            st["sched"] = FlowUniPC(int(md.get("num_steps", self.default_steps)), shift=float(md.get("shift", self.shift)))
            st["sched_walk"] = walk
        sched: FlowUniPC = st["sched"]
        gs = float(md.get("guidance_scale", 1.0))
        nb = 2 if gs != 1.0 else 1
        off = int(st.get("text_len", 0))
        cond = st.get("cond_latent")
        if cond is not None and not action:
            x[:, :1] = cond[:, :1]
        if walk == "video_sound_gen":
            return self._video_sound_step(ei, ni, ctx, x, sched, gs, nb, off, cond)
        if action:                                   # [horizon, action_dim] tokens on a 1-D position ladder
            w_in, b_in, w_out, b_out = m.action_weights(int(md.get("domain_id", 0)))
            tok = gemm.linear(x.to(m.cfg.dtype), w_in, bias=b_in) + m.action_modality_embed
            pos = (torch.arange(x.shape[0], dtype=torch.int32, device=self.device) + off)[None].repeat(3, 1)
            v = m.denoise(tok, pos, sched.timestep(), nb, ctx, w_out, b_out)
        else:
            p, grid = patchify(x, m.patch)
            tok = gemm.linear(p.to(m.cfg.dtype), m.proj_in_w, bias=m.proj_in_b)
            pos = grid_positions(*grid, self.device, (off, off, off))
            v = m.denoise(tok, pos, sched.timestep(), nb, ctx, m.proj_out_w, m.proj_out_b)
            v = torch.stack([unpatchify(v[b], grid, m.patch, m.C) for b in range(nb)])
        v = v[0] if nb == 1 else v[1] + gs * (v[0] - v[1])
        x = sched.step(v, x)
        if cond is not None and not action:
            x[:, :1] = cond[:, :1]
        return {"latents": x}

    def _video_sound_step(self, ei, ni, ctx, x, sched, gs, nb, off, cond):
        """One joint step of the [video | sound] sequence: the sound latents ride behind the video tokens as one
        token per sound latent frame, placed on the video's temporal axis at their own frame rate; both bands share
        the attention, each leaves through its own head, and ONE scheduler step updates the packed pair."""
        m, md = self.m, ni.kwargs
        n_sound = int(md["num_sound"])
        if ni.tensor_inputs.get("sound_latents"):
            xs = ni.tensor_inputs["sound_latents"][-1].to(self.device, torch.float32)
        else:       # first iteration: sound noise from the stream that follows the video noise of the same seed
            info = ei.per_request_info[ni.request_id]
            g = torch.Generator().manual_seed(int(md.get("seed", info.random_seed or 0)) + 1)
            xs = torch.randn((m.sound_dim, n_sound), generator=g).to(self.device)
        p, grid = patchify(x, m.patch)
        tok = gemm.linear(p.to(m.cfg.dtype), m.proj_in_w, bias=m.proj_in_b)
        pos = grid_positions(*grid, self.device, (off, off, off))
        stok = gemm.linear(xs.t().contiguous().to(m.cfg.dtype), m.audio_in_w, bias=m.audio_in_b) + m.audio_modality_embed
        ratio = float(md.get("sound_rate_ratio", 1.0))          # video latent frames per sound latent frame
        st_t = (torch.arange(n_sound, device=self.device, dtype=torch.float32) * ratio).floor().to(torch.int32) + off
        spos = torch.stack([st_t, torch.full_like(st_t, off), torch.full_like(st_t, off)])
        Sv = tok.shape[0]
        h = m.denoise(torch.cat([tok, stok]), torch.cat([pos, spos], dim=1), sched.timestep(), nb, ctx)
        v = gemm.linear(h[:, :Sv].reshape(nb * Sv, -1), m.proj_out_w, bias=m.proj_out_b, out_dtype=torch.float32)
        v = torch.stack([unpatchify(vb, grid, m.patch, m.C) for vb in v.reshape(nb, Sv, -1)])
        vs = gemm.linear(h[:, Sv:].reshape(nb * n_sound, -1), m.audio_out_w, bias=m.audio_out_b,
                         out_dtype=torch.float32).reshape(nb, n_sound, -1).transpose(1, 2)
        if nb == 2:
            v, vs = v[1] + gs * (v[0] - v[1]), vs[1] + gs * (vs[0] - vs[1])
        else:
            v, vs = v[0], vs[0]
        nv = x.numel()
        packed = sched.step(torch.cat([v.reshape(-1), vs.reshape(-1)]), torch.cat([x.reshape(-1), xs.reshape(-1)]))
        x, xs = packed[:nv].reshape(x.shape), packed[nv:].reshape(xs.shape)
        if cond is not None:
            x[:, :1] = cond[:, :1]
        return {"latents": x, "sound_latents": xs}

    def postprocess(self, request_id, request_info, outputs, inputs):
        outputs.pop("new_token", None)
        outputs.pop("new_token_host", None)
        return outputs


class SoundDecodeSubmodule(NodeSubmodule):
    """Sound latents [C, T] -> stereo waveform, cut to the requested number of samples, in interleaved sample order."""

    def __init__(self, dec: SoundDecoder, device):
        super().__init__(device, torch.float32)
        self.dec = dec

    def get_stateless_flavor(self):
        return "audio_codec"

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        z = ni.tensor_inputs["sound_latents"][-1].to(self.device, self.dec.conv1.weight.dtype)
        wav = self.dec.decode(z)
        n = int((ni.kwargs or {}).get("sound_samples", 0))
        if 0 < n < wav.shape[-1]:
            wav = wav[..., :n]
        return {"audio": pcm_layout(wav.float()).cpu()}


class Cosmos3Model(Model):
    name = "cosmos3"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, num_steps: int | None = None,
                 page_size: int = 128, max_num_pages: int = 512, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small = small
        if small:
            k = small_scale()
            self.cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=16 * k,
                                     intermediate_size=128 * k, vocab_size=512, qk_norm=True,
                                     mrope_sections=[2 * k, 3 * k, 3 * k],
                                     has_lm_head=False, dtype=dt)
            self.vae_cfg = tiny_vae_config(3, 4)
        else:
            self.cfg = cosmos3_nano_config(dt)
            self.vae_cfg = cosmos3_vae_config()
        self.sound_cfg = sound_decoder_config(small)
        self.action_dim = 32 if small else 64
        self.num_steps = num_steps or (3 if small else 35)
        self.page_size, self.max_num_pages = page_size, max_num_pages
        self.dtype = dt

    # ---- structure ----
    def get_graph_walk_graphs(self):
        pre_out = [GraphEdge(EMPTY_DESTINATION, "prefill_done", persist=True)]
        prefill = GraphNode("dit", {"input_ids", "neg_input_ids"}, pre_out)
        enc = GraphNode("vae_encoder", {"image"}, [GraphEdge("dit", "image_latent")])
        prefill_c = Sequential([enc, GraphNode("dit", {"input_ids", "neg_input_ids", "image_latent"}, pre_out)])

        def gen(modality, sound=False):
            names = ["latents"] + (["sound_latents"] if sound else [])
            dit = GraphNode("dit", set(names), [GraphEdge("dit", n) for n in names], enable_async_scheduling=False)
            loop_out = [GraphEdge("vae_decoder", "latents")] + ([GraphEdge("audio_decoder", "sound_latents")] if sound else [])
            tail = [GraphNode("vae_decoder", {"latents"}, [GraphEdge(EMIT_TO_CLIENT, modality, output_modality=modality)])]
            if sound:
                tail.append(GraphNode("audio_decoder", {"sound_latents"},
                                      [GraphEdge(EMIT_TO_CLIENT, "audio", output_modality="audio")]))
            return Sequential([Loop(dit, max_iters=self.num_steps, outputs=loop_out, name="denoise_loop"),
                               tail[0] if len(tail) == 1 else Parallel(tail)])
        act = GraphNode("dit", {"latents"}, [GraphEdge("dit", "latents")], enable_async_scheduling=False)
        action = Loop(act, max_iters=10, outputs=[GraphEdge(EMIT_TO_CLIENT, "latents", output_modality="action")],
                      name="denoise_loop")
        return {"prefill": prefill, "prefill_cond": prefill_c, "image_gen": gen("image"), "video_gen": gen("video"),
                "video_sound_gen": gen("video", True), "action_gen": action}

    def get_node_engine_types(self):
        return {"dit": EngineType.KV_CACHE, "vae_encoder": EngineType.STATELESS, "vae_decoder": EngineType.STATELESS,
                "audio_decoder": EngineType.STATELESS}

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=4096, max_num_pages=self.max_num_pages,
                              page_size=self.page_size, num_qo_heads=c.num_heads, nodes=["dit"], dtype=c.dtype)]

    def get_default_sharding_config(self):
        return {"dit": {"tp": True, "sp": True}}

    def get_engine_hints(self, node):
        return dict(vocab_size=8, group=self.cfg.num_heads // self.cfg.num_kv_heads, max_tokens=1 << 18,
                    n_pos_axes=3, track_seen=False, max_batch=16)

    def get_autocast_dtype(self):
        return self.dtype

    def get_output_sample_rate(self) -> int:
        return int(self.sound_cfg["sampling_rate"])

    def get_output_audio_channels(self) -> int:
        return int(self.sound_cfg["dec_out_channels"])

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "dit":
            m = Cosmos3Transformer(self.cfg, self.vae_cfg.latent_channels, tp=tp_group, sp=sp_group, device=device,
                                   sound_dim=int(self.sound_cfg["vocoder_input_dim"]), action_dim=self.action_dim,
                                   num_domains=2 if self.small else 32)
            if self.skip_weight_loading or self.model_dir is None:
                m.init_random(0)
            else:
                import os
                from .checkpoints import load_cosmos3_transformer
                load_cosmos3_transformer(m, os.path.join(self.model_dir, "transformer"))
            return Cosmos3DiTSubmodule(m, device, self.num_steps, 5.0)
        if node_name in ("vae_encoder", "vae_decoder"):
            vae = ConvVAE(self.vae_cfg).to(device=device, dtype=self.dtype).eval()
            return (VaeEncodeSubmodule(vae, device, self.dtype) if node_name == "vae_encoder"
                    else _Cosmos3VaeDecode(vae, device, self.dtype))
        if node_name == "audio_decoder":
            import os
            if (not self.skip_weight_loading and self.model_dir
                    and os.path.isdir(os.path.join(self.model_dir, "sound_tokenizer"))):
                dec = load_sound_decoder(self.model_dir, device=device, dtype=self.dtype)
            else:
                dec = seeded_init(lambda: SoundDecoder(self.sound_cfg), 11).to(device=device, dtype=self.dtype).eval()
            return SoundDecodeSubmodule(dec, device)
        raise KeyError(node_name)

    # ---- request life cycle ----
    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, negative_prompt: str = "", **kw):
        v = self.cfg.vocab_size
        enc = lambda s: torch.tensor(self.encode_text(s, v) or [0], dtype=torch.int64)  # noqa: E731
        out = {"input_ids": [enc(prompt)], "neg_input_ids": [enc(negative_prompt)]}
        if tensors and tensors.get("image"):
            out["image"] = [t.float() for t in tensors["image"]]
        return out

    def latent_shape(self, mk: dict, image: bool) -> list[int]:
        sf, tf = self.vae_cfg.spatial_factor, self.vae_cfg.temporal_factor
        H, W = int(mk.get("height", 16 if self.small else 704)), int(mk.get("width", 16 if self.small else 1280))
        frames = 1 if image else int(mk.get("num_frames", 5 if self.small else 93))
        return [self.vae_cfg.latent_channels, (frames - 1) // tf + 1, H // sf, W // sf]

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        edges = [GraphEdge("dit", "input_ids", list(input_signals["input_ids"])),
                 GraphEdge("dit", "neg_input_ids", list(input_signals["neg_input_ids"]))]
        if input_signals.get("image"):
            edges.append(GraphEdge("vae_encoder", "image", list(input_signals["image"])))
            return ForwardPassArgs({"graph_walk": "prefill_cond"}, edges)
        return ForwardPassArgs({"graph_walk": "prefill"}, edges)

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        mk = md.get("model_kwargs") or {}
        if not md["finished_walk"].startswith("prefill"):
            return ForwardPassArgs(request_done=True)
        outs = md.get("output_modalities") or ["image"]
        step_md = {k: mk[k] for k in ("shift", "seed") if k in mk}
        step_md["guidance_scale"] = float(mk.get("guidance_scale", 6.0))
        edges = [GraphEdge("dit", "latents", [])]
        if "action" in outs:
            walk, steps = "action_gen", int(mk.get("num_steps", 10))
            shape = [int(mk.get("horizon", 16)), self.action_dim]
            if "domain_id" in mk:
                step_md["domain_id"] = int(mk["domain_id"])
            step_md["num_tokens"] = shape[0]
        else:
            image = "video" not in outs
            walk = "image_gen" if image else ("video_sound_gen" if "audio" in outs else "video_gen")
            steps = int(mk.get("num_steps", self.num_steps))
            shape = self.latent_shape(mk, image)
            pt, ph, pw = (1, 2, 2)
            step_md["num_tokens"] = (shape[1] // pt) * (shape[2] // ph) * (shape[3] // pw)
            if walk == "video_sound_gen":
                # the sound track lasts as long as the video unless the request says otherwise; one latent frame per
                # hop of the sound decoder
                import math as _m
                sr = int(self.sound_cfg["sampling_rate"])
                hop = _m.prod(self.sound_cfg["dec_strides"])
                fps = float(mk.get("fps", 24))
                frames = int(mk.get("num_frames", 5 if self.small else 93))
                samples = max(1, round(float(mk.get("sound_duration", frames / fps)) * sr))
                n_sound = max(1, _m.ceil(samples / hop))
                step_md.update(num_sound=n_sound, sound_samples=samples,
                               sound_rate_ratio=(fps / self.vae_cfg.temporal_factor) / (sr / hop))
                step_md["num_tokens"] += n_sound
                edges.append(GraphEdge("dit", "sound_latents", []))
        step_md.update(num_steps=steps, latent_shape=shape)
        return ForwardPassArgs({"graph_walk": walk, "dynamic_loop_iter_counts": {"denoise_loop": steps}},
                               edges, step_metadata=step_md)

    def postprocess(self, output, modality, request_kwargs):
        from ..api_server.media_io import float_to_pcm16, frames_to_video, tensor_to_png
        t = output if isinstance(output, torch.Tensor) else output[-1]
        if modality == "image":
            return tensor_to_png(t[:, 0] if t.dim() == 4 else t)
        if modality == "video":
            return frames_to_video(t.permute(1, 0, 2, 3), fps=float(request_kwargs.get("fps", 24)))[0]
        if modality == "audio":
            return float_to_pcm16(t)                # [samples, channels]: interleaved PCM
        return t.float().numpy().tobytes()          # action chunk: raw float32 [horizon, action_dim]


class _Cosmos3VaeDecode(VaeDecodeSubmodule):
    def forward(self, graph_walk, engine_inputs, ni, **kw):
        out = super().forward(graph_walk, engine_inputs, ni, **kw)
        px = out.pop("video")
        return {"image" if graph_walk == "image_gen" else "video": px}


class Cosmos3SuperModel(Cosmos3Model):
    """Larger backbone (Qwen3-14B-class shape); meant for tp2 / tp4 / tp2 x sp2 placements."""
    name = "cosmos3_super"

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        if not self.small:
            self.cfg = DecoderConfig(hidden_size=5120, num_layers=40, num_heads=40, num_kv_heads=8, head_dim=128,
                                     intermediate_size=17408, vocab_size=151936, rope_theta=1e6, qk_norm=True,
                                     mrope_sections=[24, 20, 20], has_lm_head=False, dtype=self.dtype)


class Cosmos3DroidModel(Cosmos3Model):
    """Robot-policy variant: requests default to an action chunk conditioned on the camera image."""
    name = "cosmos3_droid"

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = dict(partition_metadata)
        if not md.get("output_modalities") or md["output_modalities"] == ["text"]:
            md["output_modalities"] = ["action"]
        return super().get_partition_forward_pass_args(partition_name, md, persist_signals, incoming_connections)
