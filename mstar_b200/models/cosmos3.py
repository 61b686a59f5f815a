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
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .codec import Code2Wav
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
                 tp: CommGroup | None = None, sp: CommGroup | None = None, device="cpu"):
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
        self.act_in_w, self.act_out_w = _param((H, action_dim), dt, device), _param((action_dim, H), dt, device)
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

    def time_embed(self, t: torch.Tensor) -> torch.Tensor:
        e = sinusoidal_embedding(t, 256).to(self.cfg.dtype)
        e = gemm.linear(e, self.t1_w, bias=self.t1_b)
        return gemm.linear(torch.nn.functional.silu(e.float()).to(e.dtype), self.t2_w, bias=self.t2_b)

    def denoise(self, tokens: torch.Tensor, positions: torch.Tensor, t: float, n_branches: int, prefix_ctx,
                out_w, out_b=None) -> torch.Tensor:
        """tokens: [S, H] embedded noisy tokens of ONE request; runs ``n_branches`` guidance branches packed as
        [branch0 | branch1 | ...] and returns [n_branches, S, out] fp32."""
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
            h = gather_sequence(h, self.sp, S_tot)
        else:
            h = self.gen(x, pos, plan, prefix_ctx=prefix_ctx, S_total=S_tot)
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
        if action:                                   # [horizon, action_dim] tokens on a 1-D position ladder
            tok = gemm.linear(x.to(m.cfg.dtype), m.act_in_w)
            pos = (torch.arange(x.shape[0], dtype=torch.int32, device=self.device) + off)[None].repeat(3, 1)
            v = m.denoise(tok, pos, sched.timestep(), nb, ctx, m.act_out_w)
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

    def postprocess(self, request_id, request_info, outputs, inputs):
        outputs.pop("new_token", None)
        outputs.pop("new_token_host", None)
        return outputs


class AudioDecodeSubmodule(NodeSubmodule):
    """Sound track from the video latents' temporal envelope through a code-to-waveform stack."""

    def __init__(self, dec: Code2Wav, device, n_codes: int):
        super().__init__(device, torch.float32)
        self.dec, self.n_codes = dec, n_codes

    def get_stateless_flavor(self):
        return "audio_codec"

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        z = ni.tensor_inputs["latents"][-1].float()
        env = z.mean(dim=(0, 2, 3))                                   # one value per latent frame
        codes = ((env - env.min()) / (env.max() - env.min() + 1e-6) * (self.n_codes - 1)).long()
        with torch.no_grad():
            wav = self.dec(codes[None, None].to(self.device))[0]
        return {"audio": wav.float().cpu().reshape(-1)}


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
            dit = GraphNode("dit", {"latents"}, [GraphEdge("dit", "latents")], enable_async_scheduling=False)
            loop_out = [GraphEdge("vae_decoder", "latents")] + ([GraphEdge("audio_decoder", "latents")] if sound else [])
            tail = [GraphNode("vae_decoder", {"latents"}, [GraphEdge(EMIT_TO_CLIENT, modality, output_modality=modality)])]
            if sound:
                tail.append(GraphNode("audio_decoder", {"latents"}, [GraphEdge(EMIT_TO_CLIENT, "audio", output_modality="audio")]))
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

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "dit":
            m = Cosmos3Transformer(self.cfg, self.vae_cfg.latent_channels, tp=tp_group, sp=sp_group, device=device)
            if self.skip_weight_loading or self.model_dir is None:
                m.init_random(0)
            else:
                from .loader import load_named_tensors
                load_named_tensors(m, self.model_dir)
            return Cosmos3DiTSubmodule(m, device, self.num_steps, 5.0)
        if node_name in ("vae_encoder", "vae_decoder"):
            vae = ConvVAE(self.vae_cfg).to(device=device, dtype=self.dtype).eval()
            return (VaeEncodeSubmodule(vae, device, self.dtype) if node_name == "vae_encoder"
                    else _Cosmos3VaeDecode(vae, device, self.dtype))
        if node_name == "audio_decoder":
            kw = (dict(n_codebooks=1, codebook_size=64, dim=16, rates=(2, 2), channels=32) if self.small
                  else dict(n_codebooks=1))
            return AudioDecodeSubmodule(Code2Wav(**kw).to(device).eval(), device, kw.get("codebook_size", 2048))
        raise KeyError(node_name)

    # ---- request life cycle ----
    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, negative_prompt: str = "", **kw):
        v = self.cfg.vocab_size
        enc = lambda s: torch.tensor([b % v for b in (s or "").encode("utf-8")] or [0], dtype=torch.int64)  # noqa: E731
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
        if "action" in outs:
            walk, steps = "action_gen", int(mk.get("num_steps", 10))
            shape = [int(mk.get("horizon", 16)), 32]
            step_md["num_tokens"] = shape[0]
        else:
            image = "video" not in outs
            walk = "image_gen" if image else ("video_sound_gen" if "audio" in outs else "video_gen")
            steps = int(mk.get("num_steps", self.num_steps))
            shape = self.latent_shape(mk, image)
            pt, ph, pw = (1, 2, 2)
            step_md["num_tokens"] = (shape[1] // pt) * (shape[2] // ph) * (shape[3] // pw)
        step_md.update(num_steps=steps, latent_shape=shape)
        return ForwardPassArgs({"graph_walk": walk, "dynamic_loop_iter_counts": {"denoise_loop": steps}},
                               [GraphEdge("dit", "latents", [])], step_metadata=step_md)

    def postprocess(self, output, modality, request_kwargs):
        from ..api_server.media_io import float_to_pcm16, frames_to_video, tensor_to_png
        t = output if isinstance(output, torch.Tensor) else output[-1]
        if modality == "image":
            return tensor_to_png(t[:, 0] if t.dim() == 4 else t)
        if modality == "video":
            return frames_to_video(t.permute(1, 0, 2, 3), fps=float(request_kwargs.get("fps", 24)))[0]
        if modality == "audio":
            return float_to_pcm16(t)
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
