"""Wan2.2-TI2V-5B class text/image-to-video generator: UMT5 text encoder, causal 3D VAE (48 latent channels, 16x
spatial, 4x temporal), AdaLN DiT (30 layers, hidden 3072, 24 heads), UniPC sampler, classifier-free guidance as a
batch of two sequences through one forward.

Walks: ``encode_text`` (prompt + negative prompt -> text context, kept by the conductor), ``encode_image``
(image-to-video: first frame -> latent), ``video_gen`` / ``video_gen_i2v`` (Loop ``denoise_loop`` around ``dit``,
then ``vae_decoder`` emits the video). The sampler state lives with the request inside the dit node; the latents
travel on the loop-back edge.

Reference counterparts: mstar/model/wan22/wan22_model.py (walks, state machine), submodules.py (text_encoder,
vae_encoder, dit, vae_decoder nodes), components/dit.py, components/unipc.py, config.py.
"""
from __future__ import annotations

import torch

from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop, Sequential
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .dit import AdaLNDiT, DiTConfig, wan22_5b_config
from .encoders import T5Encoder
from .schedulers import FlowUniPC
from .submodule_base import NodeSubmodule
from .vae import ConvVAE, VAEConfig, tiny_vae_config, wan22_vae_config


class TextEncoderSubmodule(NodeSubmodule):
    def __init__(self, enc: T5Encoder, device, text_len: int):
        super().__init__(device, enc.c.dtype)
        self.enc, self.text_len = enc, text_len

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        outs = {}
        for key, edge in (("input_ids", "text_context"), ("neg_input_ids", "neg_context")):
            ids = torch.cat([t.reshape(-1) for t in ni.tensor_inputs.get(key, [])] or [torch.zeros(1, dtype=torch.int64)])
            ids = ids[:self.text_len].to(self.device)
            with torch.no_grad():
                outs[edge] = self.enc(ids)
        return outs


class VaeEncodeSubmodule(NodeSubmodule):
    def __init__(self, vae: ConvVAE, device, dtype):
        super().__init__(device, dtype)
        self.vae = vae

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        img = ni.tensor_inputs["image"][0].to(self.device, self.dtype)          # [3, H, W] in [-1, 1]
        x = img[None, :, None] if self.vae.cfg.dims == 3 else img[None]
        return {"image_latent": self.vae.encode(x)[0].float()}


class VaeDecodeSubmodule(NodeSubmodule):
    def __init__(self, vae: ConvVAE, device, dtype, tile: int = 0, out_edge: str = "video"):
        super().__init__(device, dtype)
        self.vae, self.tile, self.out_edge = vae, tile, out_edge

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        z = ni.tensor_inputs["latents"][-1].to(self.device, self.dtype)
        px = self.vae.decode(z[None], tile=self.tile)[0]
        return {self.out_edge: px.float().cpu()}


class WanDiTSubmodule(NodeSubmodule):
    """One denoising step per forward. Per-request state: sampler, projected text K/V of both guidance branches,
    image latent of image-to-video requests."""

    def __init__(self, dit: AdaLNDiT, device, default_steps: int, shift: float):
        super().__init__(device, dit.cfg.dtype)
        self.dit, self.default_steps, self.shift = dit, default_steps, shift

    def can_batch(self, graph_walk):
        return False

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        st = engine_inputs.per_request_states[ni.request_id]
        md = ni.kwargs
        if ni.tensor_inputs.get("latents"):
            x = ni.tensor_inputs["latents"][-1].to(self.device, torch.float32)   # [C, F, H, W]
        else:                                        # first step: the request's seed makes the noise
            info = engine_inputs.per_request_info[ni.request_id]
            g = torch.Generator().manual_seed(int(md.get("seed", info.random_seed or 0)))
            x = torch.randn(tuple(md["latent_shape"]), generator=g).to(self.device)
        if "sched" not in st:
            st["sched"] = FlowUniPC(int(md.get("num_steps", self.default_steps)), shift=float(md.get("shift", self.shift)))
            st["gs"] = float(md.get("guidance_scale", 5.0))
            ctxs = [ni.tensor_inputs["text_context"][0].to(self.device)]
            if st["gs"] != 1.0:
                ctxs.append(ni.tensor_inputs["neg_context"][0].to(self.device))
            st["ctx_lens"] = [c.shape[0] for c in ctxs]
            st["ctx_kv"] = self.dit.encode_context(torch.cat(ctxs))
            st["img"] = ni.tensor_inputs["image_latent"][0].to(self.device, torch.float32) \
                if ni.tensor_inputs.get("image_latent") else None
        sched: FlowUniPC = st["sched"]
        B = len(st["ctx_lens"])
        t = sched.timestep()
        Fp = x.shape[1] // self.dit.cfg.patch_size[0]
        ts = torch.full((B, Fp), t, device=self.device)
        if st["img"] is not None:                    # the first latent frame is the (clean) conditioning image
            x[:, :1] = st["img"][:, :1]
            ts[:, 0] = 0.0
        v = self.dit(x[None].expand(B, -1, -1, -1, -1), ts, st["ctx_kv"], st["ctx_lens"])
        v = v[0] if B == 1 else v[1] + st["gs"] * (v[0] - v[1])
        x = sched.step(v, x)
        if st["img"] is not None:
            x[:, :1] = st["img"][:, :1]
        return {"latents": x}


class Wan22Model(Model):
    name = "wan22"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, num_steps: int | None = None,
                 vae_tile: int = 0, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        self.small = small
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        if small:
            k = small_scale()
            self.dit_cfg = DiTConfig(hidden_size=64 * k, num_layers=2, num_heads=4, head_dim=16 * k, ffn_dim=128 * k,
                                     in_channels=4, out_channels=4, text_dim=32 * k, text_len=16, dtype=dt,
                                     rope_axes=(4 * k, 6 * k, 6 * k))
            self.vae_cfg = tiny_vae_config(3, 4)
            self.text = dict(vocab_size=512, hidden=32 * k, layers=1, heads=2, head_dim=16 * k, ffn=64 * k)
        else:
            self.dit_cfg = wan22_5b_config()
            self.vae_cfg = wan22_vae_config()
            self.text = dict()
        self.num_steps = num_steps or (3 if small else 50)
        self.vae_tile = vae_tile
        self.dtype = dt

    # ---- structure ----
    def get_graph_walk_graphs(self):
        enc_t = GraphNode("text_encoder", {"input_ids", "neg_input_ids"},
                          [GraphEdge(EMPTY_DESTINATION, "text_context", persist=True),
                           GraphEdge(EMPTY_DESTINATION, "neg_context", persist=True)])
        enc_i = GraphNode("vae_encoder", {"image"}, [GraphEdge(EMPTY_DESTINATION, "image_latent", persist=True)])

        def gen(i2v):
            ins = {"latents", "text_context", "neg_context"} | ({"image_latent"} if i2v else set())
            dit = GraphNode("dit", ins, [GraphEdge("dit", "latents")], enable_async_scheduling=False)
            dec = GraphNode("vae_decoder", {"latents"}, [GraphEdge(EMIT_TO_CLIENT, "video", output_modality="video")])
            return Sequential([Loop(dit, max_iters=self.num_steps, outputs=[GraphEdge("vae_decoder", "latents")],
                                    name="denoise_loop"), dec])
        from ..graph.ir import Parallel
        return {"encode_text": enc_t, "encode_text_image": Parallel([enc_t, enc_i]), "video_gen": gen(False),
                "video_gen_i2v": gen(True)}

    def get_node_engine_types(self):
        return {n: EngineType.STATELESS for n in ("text_encoder", "vae_encoder", "dit", "vae_decoder")}

    def get_kv_cache_config(self):
        return []

    def get_default_sharding_config(self):
        return {"dit": {"tp": True, "sp": True}}

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "text_encoder":
            enc = T5Encoder(dtype=self.dtype, device=device, **self.text)
            return TextEncoderSubmodule(self._init(enc, "text_encoder"), device, self.dit_cfg.text_len)
        if node_name in ("vae_encoder", "vae_decoder"):
            vae = ConvVAE(self.vae_cfg).to(device=device, dtype=self.dtype).eval()
            return (VaeEncodeSubmodule(vae, device, self.dtype) if node_name == "vae_encoder"
                    else VaeDecodeSubmodule(vae, device, self.dtype, self.vae_tile))
        if node_name == "dit":
            dit = AdaLNDiT(self.dit_cfg, device, tp=tp_group, sp=sp_group)
            return WanDiTSubmodule(self._init(dit, "transformer"), device, self.num_steps, 5.0)
        raise KeyError(node_name)

    def _init(self, module, component: str):
        """Random-init weights, or the published (diffusers) checkpoint: ``model_dir/transformer`` in the
        ``WanTransformer3DModel`` layout, ``model_dir/text_encoder`` in the Hugging Face UMT5 layout. Both loads are
        strict. A directory without those components is read as tensors saved under this library's own names."""
        if self.skip_weight_loading or self.model_dir is None:
            return module.init_random(0)
        import os
        sub = os.path.join(self.model_dir, component)
        if os.path.isdir(sub):
            from .checkpoints import load_t5_encoder, load_wan22_transformer
            (load_wan22_transformer if component == "transformer" else load_t5_encoder)(module, sub)
            return module
        from .loader import load_named_tensors
        load_named_tensors(module, self.model_dir)
        return module

    # ---- request life cycle ----
    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, negative_prompt: str = "", **kw):
        v = self.text.get("vocab_size", 256384)
        enc = lambda s: torch.tensor(self.encode_text(s, v, default=" ") + [1], dtype=torch.int64)  # noqa: E731
        out = {"input_ids": [enc(prompt)], "neg_input_ids": [enc(negative_prompt)]}
        if tensors and tensors.get("image"):
            out["image"] = [t.float() for t in tensors["image"]]
        return out

    def latent_shape(self, mk: dict) -> tuple[int, int, int, int]:
        sf, tf = self.vae_cfg.spatial_factor, self.vae_cfg.temporal_factor
        H, W = int(mk.get("height", 704 if not self.small else 16)), int(mk.get("width", 1280 if not self.small else 16))
        frames = int(mk.get("num_frames", 121 if not self.small else 3))
        return (self.dit_cfg.in_channels, (frames - 1) // tf + 1, H // sf, W // sf)

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        edges = [GraphEdge("text_encoder", "input_ids", list(input_signals["input_ids"])),
                 GraphEdge("text_encoder", "neg_input_ids", list(input_signals["neg_input_ids"]))]
        if input_signals.get("image"):
            edges.append(GraphEdge("vae_encoder", "image", list(input_signals["image"])))
            return ForwardPassArgs({"graph_walk": "encode_text_image"}, edges)
        return ForwardPassArgs({"graph_walk": "encode_text"}, edges)

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        mk = md.get("model_kwargs") or {}
        if md["finished_walk"] in ("encode_text", "encode_text_image"):
            i2v = bool(persist_signals.get("image_latent"))
            steps = int(mk.get("num_steps", self.num_steps))
            edges = [GraphEdge("dit", "latents", []), GraphEdge("dit", "text_context", persist_signals["text_context"]),
                     GraphEdge("dit", "neg_context", persist_signals["neg_context"])]
            if i2v:
                edges.append(GraphEdge("dit", "image_latent", persist_signals["image_latent"]))
            step_md = {k: mk[k] for k in ("guidance_scale", "shift", "seed") if k in mk}
            step_md.update(num_steps=steps, latent_shape=list(self.latent_shape(mk)))
            return ForwardPassArgs({"graph_walk": "video_gen_i2v" if i2v else "video_gen",
                                    "dynamic_loop_iter_counts": {"denoise_loop": steps}}, edges, step_metadata=step_md)
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        from ..api_server.media_io import frames_to_video
        vid = output if isinstance(output, torch.Tensor) else output[-1]          # [3, T, H, W] in [-1, 1]
        return frames_to_video(vid.permute(1, 0, 2, 3), fps=float(request_kwargs.get("fps", 24)))[0]
