"""V-JEPA 2 class video world model: a ViT video encoder (tubelets of 2 frames x 16 x 16 pixels), a masked-token
predictor, and (V-JEPA 2-AC) an action-conditioned predictor that rolls future frame embeddings forward from
actions and end-effector states, with an energy scorer for model-predictive control.

Nodes (all stateless): ``video_encoder``, ``predictor``.
Walks: ``prefill_video`` (encode, then predict the embeddings of the masked tubelets),
``prefill_video_encoder_only`` (embeddings out), ``rollout`` (encode the context frame, then Loop ``rollout_loop``
of the action-conditioned predictor; every step's embeddings are accumulated), ``mpc_score`` (K candidate action
sequences rolled out as one batch, L1 energy to the goal embedding per candidate).
The transformer stacks run through a piecewise CUDA-graph runner: blocks are captured per shape, the
mask-dependent gather / scatter around them stays eager.

Reference counterparts: mstar/model/vjepa2/vjepa2_model.py (1116 lines), submodules.py (1481; piecewise graphs
:919-953), components/ac_predictor.py (578), components/layers.py, weight_loader.py (373).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..engine.piecewise_graph import PiecewiseCudaGraphRunner
from ..graph.ir import EMIT_TO_CLIENT, GraphEdge, GraphNode, Loop, Sequential
from ..ops import gemm
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .encoders import EncoderConfig, TransformerEncoder
from .submodule_base import NodeSubmodule


def _p(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


def rope3d_tables(ids: torch.Tensor, grid_hw: tuple[int, int], head_dim: int):
    """Cosine / sine tables [T, 1, 3s] of the published rotary embedding of V-JEPA 2 for tokens at flat tubelet
    indices ``ids`` (frame-major, then rows, then columns): the head is cut into three bands of s = 2 * ((D // 3) // 2)
    channels for the frame, row and column position (what is left over is not rotated); the angle of channel j of a
    band is position x 10000^(-(j mod s/2) / (s/2)) — the angle table is tiled over the band, not repeated per pair
    (transformers/models/vjepa2/modeling_vjepa2.py: rotate_queries_or_keys)."""
    h, w = grid_hw
    ids = ids.long()
    frame = ids // (h * w)
    row = (ids - frame * h * w) // w
    col = ids - frame * h * w - row * w
    s = 2 * ((head_dim // 3) // 2)
    omega = 1.0 / 10000 ** (torch.arange(s // 2, dtype=torch.float32, device=ids.device) / (s / 2.0))
    ang = torch.cat([(p.float()[:, None] * omega).repeat(1, 2) for p in (frame, row, col)], dim=-1)     # [T, 3s]
    return torch.cos(ang)[:, None].contiguous(), torch.sin(ang)[:, None].contiguous()


def rope3d_apply(cs: torch.Tensor, sn: torch.Tensor):
    """The rotation for [T, heads, D] tensors: inside a band adjacent channels (2i, 2i+1) form the rotated pair."""
    n = cs.shape[-1]

    def apply(x):
        xf = x.float()
        r = xf[..., :n]
        pair = r.unflatten(-1, (-1, 2))
        y = torch.stack((-pair[..., 1], pair[..., 0]), dim=-1).flatten(-2)
        return torch.cat([r * cs + y * sn, xf[..., n:]], dim=-1).to(x.dtype)
    return apply


def rope3d(ids: torch.Tensor, grid_hw: tuple[int, int], head_dim: int):
    return rope3d_apply(*rope3d_tables(ids, grid_hw, head_dim))


class VJepa2Encoder(nn.Module):
    """ViT over tubelets (2 frames x patch x patch pixels) with the 3-axis rotary embedding and no position table;
    pre-LN blocks, exact GELU, final LayerNorm. Reference: mstar/model/vjepa2/components/vit_encoder.py."""

    def __init__(self, c: EncoderConfig, patch: int = 16, tubelet: int = 2, in_channels: int = 3, device="cpu"):
        super().__init__()
        self.c, self.patch, self.tp = c, patch, tubelet
        pdim = in_channels * tubelet * patch * patch
        self.patch_w, self.patch_b = _p((c.hidden_size, pdim), c.dtype, device), _p((c.hidden_size,), c.dtype, device)
        self.enc = TransformerEncoder(c, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.patch_w.data.copy_((torch.randn(self.patch_w.shape, generator=g) / math.sqrt(self.patch_w.shape[-1])).to(self.c.dtype))
        self.patch_b.data.zero_()
        self.enc.init_random(seed + 1)
        return self

    def patches(self, vid: torch.Tensor):
        """[C, T, H, W] clip (or [C, H, W] image, repeated over the tubelet) -> ([t*h*w, C*tp*p*p], (t, h, w))."""
        if vid.dim() == 3:
            vid = vid[:, None].expand(-1, self.tp, -1, -1)
        if vid.shape[1] < self.tp:
            vid = vid.repeat(1, self.tp, 1, 1)
        C, T, H, W = vid.shape
        p, tp = self.patch, self.tp
        t, h, w = T // tp, H // p, W // p
        x = vid[:, :t * tp, :h * p, :w * p].reshape(C, t, tp, h, p, w, p).permute(1, 3, 5, 0, 2, 4, 6)
        return x.reshape(t * h * w, C * tp * p * p), (t, h, w)

    def forward(self, videos: list[torch.Tensor]):
        """Returns (features [sum tokens, hidden], tokens per clip, grids)."""
        toks, grids, ids = [], [], []
        for v in videos:
            pt, g = self.patches(v.to(self.c.dtype))
            toks.append(pt), grids.append(g)
            ids.append(torch.arange(pt.shape[0], device=pt.device))
        x = gemm.linear(torch.cat(toks).contiguous(), self.patch_w, bias=self.patch_b)
        lens = [g[0] * g[1] * g[2] for g in grids]
        if len({(g[1], g[2]) for g in grids}) != 1:
            raise ValueError("clips of one batch must share their frame size")
        rope = rope3d(torch.cat(ids), (grids[0][1], grids[0][2]), self.c.head_dim)
        return self.enc(x, lens, rope=rope), lens, grids


class MaskedPredictor(nn.Module):
    """Narrow transformer over [context tokens ‖ mask tokens at the target positions] -> embeddings of the targets;
    positions enter through the same 3-axis rotary embedding as in the encoder (the published predictor sorts the
    tokens by position first, which changes nothing for full attention). Reference:
    mstar/model/vjepa2/components/predictor.py."""

    def __init__(self, enc_dim: int, c: EncoderConfig, device, num_mask_tokens: int = 10):
        super().__init__()
        self.c = c
        self.inp_w, self.inp_b = _p((c.hidden_size, enc_dim), c.dtype, device), _p((c.hidden_size,), c.dtype, device)
        self.out_w, self.out_b = _p((enc_dim, c.hidden_size), c.dtype, device), _p((enc_dim,), c.dtype, device)
        self.mask_tokens = _p((num_mask_tokens, c.hidden_size), c.dtype, device)
        self.blocks = TransformerEncoder(c, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for p in (self.inp_w, self.out_w, self.mask_tokens):
            p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1])).to(p.dtype))
        self.inp_b.data.zero_(), self.out_b.data.zero_()
        self.blocks.init_random(seed + 1)
        return self

    def forward(self, ctx_tokens, ctx_idx, tgt_idx, runner: PiecewiseCudaGraphRunner, grid_hw: tuple[int, int],
                mask_index: int = 1):
        x = gemm.linear(ctx_tokens, self.inp_w, bias=self.inp_b)
        m = self.mask_tokens[mask_index % self.mask_tokens.shape[0]].expand(tgt_idx.numel(), -1)
        seq = torch.cat([x, m.to(x.dtype)]).contiguous()
        n = seq.shape[0]
        # the position tables are INPUTS of the captured piece: a replay for other masks of the same size must rotate
        # by its own positions
        cs, sn = rope3d_tables(torch.cat([ctx_idx, tgt_idx]), grid_hw, self.c.head_dim)
        h = runner.run("predictor_blocks", lambda s_, c_, n_: self.blocks(s_, [n], rope=rope3d_apply(c_, n_)), seq, cs, sn)
        return gemm.linear(h[x.shape[0]:].contiguous(), self.out_w, bias=self.out_b)


class ActionConditionedPredictor(nn.Module):
    """Per time step: the frame's patch embeddings plus one action token and one state token; block-causal over
    time (a frame sees itself and the past). Predicts the next frame's patch embeddings."""

    def __init__(self, enc_dim: int, c: EncoderConfig, action_dim: int, state_dim: int, device):
        super().__init__()
        self.c = c
        self.inp = _p((c.hidden_size, enc_dim), c.dtype, device)
        self.act = _p((c.hidden_size, action_dim), c.dtype, device)
        self.state = _p((c.hidden_size, state_dim), c.dtype, device)
        self.out = _p((enc_dim, c.hidden_size), c.dtype, device)
        self.blocks = TransformerEncoder(c, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for p in (self.inp, self.act, self.state, self.out):
            p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1])).to(p.dtype))
        self.blocks.init_random(seed + 1)
        return self

    def step(self, frames: torch.Tensor, actions: torch.Tensor, states: torch.Tensor, runner) -> torch.Tensor:
        """frames [B, T, P, E] (history incl. current), actions [B, T, A], states [B, T, S] -> next frame [B, P, E].
        The history of every candidate is its own attention sequence (full attention inside; the history only holds
        the past, so nothing from the future can leak)."""
        B, T, P, E = frames.shape
        dt = self.c.dtype
        x = gemm.linear(frames.reshape(B * T * P, E).to(dt), self.inp).reshape(B, T, P, -1)
        a = gemm.linear(actions.reshape(B * T, -1).to(dt), self.act).reshape(B, T, 1, -1)
        s = gemm.linear(states.reshape(B * T, -1).to(dt), self.state).reshape(B, T, 1, -1)
        seq = torch.cat([a, s, x], dim=2).reshape(B * T * (P + 2), -1).contiguous()
        L = T * (P + 2)
        h = runner.run(f"ac_blocks_{B}x{L}", lambda z: self.blocks(z, [L] * B), seq)
        last = h.reshape(B, T, P + 2, -1)[:, -1, 2:].reshape(B * P, -1).contiguous()
        return gemm.linear(last, self.out).reshape(B, P, E)


class VideoEncoderSubmodule(NodeSubmodule):
    def __init__(self, enc: VJepa2Encoder, device):
        super().__init__(device, enc.c.dtype)
        self.enc = enc

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        vids = [t.to(self.device) for t in ni.tensor_inputs.get("video", []) + ni.tensor_inputs.get("image", [])]
        feats, lens, grids = self.enc(vids)
        out = {"video_features": feats, "grid": torch.tensor(grids[0], dtype=torch.int64)}
        if len(vids) > 1:          # second clip / image = the goal of a planning request
            out["video_features"], out["goal_features"] = feats[:lens[0]], feats[lens[0]:]
        return out


class PredictorSubmodule(NodeSubmodule):
    def __init__(self, masked: MaskedPredictor, ac: ActionConditionedPredictor | None, device, use_graphs=None):
        super().__init__(device, masked.c.dtype)
        self.masked, self.ac = masked, ac
        self.runner = PiecewiseCudaGraphRunner(use_graphs)

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        md = ni.kwargs
        st = engine_inputs.per_request_states[ni.request_id]
        if graph_walk == "prefill_video":
            grid = [int(x) for x in ni.tensor_inputs["grid"][0].tolist()]
            feats = ni.tensor_inputs["video_features"][0].to(self.device)
            n = feats.shape[0]
            g = torch.Generator().manual_seed(int(md.get("seed", 0)))
            perm = torch.randperm(n, generator=g)
            k = max(1, int(n * float(md.get("mask_ratio", 0.5))))
            tgt, ctx = perm[:k].sort().values.to(self.device), perm[k:].sort().values.to(self.device)
            pred = self.masked(feats[ctx].contiguous(), ctx, tgt, self.runner, (grid[1], grid[2]))
            return {"embeddings": pred.float().cpu(), "target_index": tgt.cpu()}
        grid = [int(x) for x in ni.tensor_inputs["grid"][0].tolist()]
        P = grid[1] * grid[2]
        acts = ni.tensor_inputs["actions"][0].to(self.device).float()                 # [K, T, A] or [T, A]
        acts = acts[None] if acts.dim() == 2 else acts
        K, T = acts.shape[0], acts.shape[1]
        state0 = (ni.tensor_inputs["state"][0].to(self.device).float().reshape(1, -1)
                  if ni.tensor_inputs.get("state") else torch.zeros(1, self.ac.state.shape[1], device=self.device))
        if graph_walk == "rollout":
            if ni.tensor_inputs.get("frames"):
                frames = ni.tensor_inputs["frames"][-1].to(self.device)
                i = st["i"]
            else:
                frames = ni.tensor_inputs["video_features"][0].to(self.device)[-P:].reshape(1, 1, P, -1)
                i = st["i"] = 0
            states = state0[:, None].expand(1, frames.shape[1], -1)
            nxt = self.ac.step(frames, acts[:1, :i + 1], states, self.runner)
            st["i"] = i + 1
            return {"frames": torch.cat([frames, nxt[:, None].to(frames.dtype)], dim=1), "embeddings": nxt[0].float().cpu()}
        # mpc_score: all candidates in one batch, horizon T
        cur = ni.tensor_inputs["video_features"][0].to(self.device)[-P:].reshape(1, 1, P, -1).expand(K, -1, -1, -1)
        goal = ni.tensor_inputs["goal_features"][0].to(self.device)[-P:].float()
        frames = cur
        for t in range(T):
            states = state0[:, None].expand(K, frames.shape[1], -1)
            nxt = self.ac.step(frames, acts[:, :t + 1], states, self.runner)
            frames = torch.cat([frames, nxt[:, None].to(frames.dtype)], dim=1)
        energy = (frames[:, -1].float() - goal[None]).abs().mean(dim=(1, 2))
        return {"energy": energy.cpu(), "best_action": acts[energy.argmin()].cpu()}


class VJepa2Model(Model):
    name = "vjepa2"
    action_conditioned = False

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype = small, dt
        k = small_scale()
        if small:
            self.enc_cfg, self.patch = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, act="gelu_erf", dtype=dt), 4
            self.pred_cfg = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, act="gelu_erf", dtype=dt)
        else:      # ViT-L encoder, 12-layer 384-wide predictor
            self.enc_cfg, self.patch = EncoderConfig(1024, 24, 16, 64, 4096, act="gelu_erf", dtype=dt), 16
            self.pred_cfg = EncoderConfig(384, 12, 12, 32, 1536, act="gelu_erf", dtype=dt)
        self.ac_cfg = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, dtype=dt) if small else EncoderConfig(1024, 24, 16, 64, 4096, dtype=dt)
        self.action_dim, self.state_dim = 7, 7

    def get_graph_walk_graphs(self):
        def enc(extra=()):
            return GraphNode("video_encoder", {"video"}, [GraphEdge("predictor", n) for n in ("video_features", "grid") + tuple(extra)])
        emb = [GraphEdge(EMIT_TO_CLIENT, "embeddings", output_modality="embeddings")]
        walks = {
            "prefill_video": Sequential([enc(), GraphNode("predictor", {"video_features", "grid"}, emb)]),
            "prefill_video_encoder_only": GraphNode("video_encoder", {"video"},
                                                    [GraphEdge(EMIT_TO_CLIENT, "video_features", output_modality="embeddings")]),
        }
        if self.action_conditioned:
            step = GraphNode("predictor", {"video_features", "grid", "actions", "state", "frames"},
                             [GraphEdge("predictor", "frames"), GraphEdge("__empty_destination__", "embeddings")],
                             enable_async_scheduling=False)
            walks["rollout"] = Sequential([enc(), Loop(step, max_iters=64, name="rollout_loop",
                                                       accumulated_outputs=[GraphEdge(EMIT_TO_CLIENT, "embeddings",
                                                                                      output_modality="embeddings")])])
            walks["mpc_score"] = Sequential([enc(("goal_features",)),
                                             GraphNode("predictor", {"video_features", "grid", "goal_features", "actions", "state"},
                                                       [GraphEdge(EMIT_TO_CLIENT, "energy", output_modality="energy"),
                                                        GraphEdge(EMIT_TO_CLIENT, "best_action", output_modality="action")])])
        return walks

    def get_node_engine_types(self):
        return {"video_encoder": EngineType.STATELESS, "predictor": EngineType.STATELESS}

    def get_kv_cache_config(self):
        return []

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "video_encoder":
            enc = VJepa2Encoder(self.enc_cfg, patch=self.patch, tubelet=2, device=device).init_random(0)
            if not (self.skip_weight_loading or self.model_dir is None):
                from .checkpoints import load_vjepa2_encoder
                load_vjepa2_encoder(enc, self.model_dir)
            return VideoEncoderSubmodule(enc, device)
        if node_name == "predictor":
            masked = MaskedPredictor(self.enc_cfg.hidden_size, self.pred_cfg, device).init_random(1)
            if not (self.skip_weight_loading or self.model_dir is None):
                from .checkpoints import load_vjepa2_predictor
                load_vjepa2_predictor(masked, self.model_dir)
            ac = (ActionConditionedPredictor(self.enc_cfg.hidden_size, self.ac_cfg, self.action_dim, self.state_dim,
                                             device).init_random(2) if self.action_conditioned else None)
            return PredictorSubmodule(masked, ac, device)
        raise KeyError(node_name)

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        vids = [t.float() for t in (tensors.get("video") or []) + (tensors.get("image") or [])]
        if not vids:
            raise ValueError("a video (or image) input is required")
        out = {"video": vids}
        for k in ("actions", "state"):
            if tensors.get(k):
                out[k] = [tensors[k][0].float()]
        return out

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        mk = model_kwargs or {}
        edges = [GraphEdge("video_encoder", "video", list(input_signals["video"]))]
        task = mk.get("task", "rollout" if self.action_conditioned and input_signals.get("actions") else "predict")
        smd = {k: mk[k] for k in ("seed", "mask_ratio") if k in mk}
        if task in ("rollout", "mpc") and self.action_conditioned:
            edges.append(GraphEdge("predictor", "actions", list(input_signals["actions"])))
            edges.append(GraphEdge("predictor", "state", list(input_signals.get("state", []))))
            if task == "rollout":
                edges.append(GraphEdge("predictor", "frames", []))
                n = int(mk.get("horizon", 4))
                return ForwardPassArgs({"graph_walk": "rollout", "dynamic_loop_iter_counts": {"rollout_loop": n}}, edges,
                                       step_metadata=smd)
            return ForwardPassArgs({"graph_walk": "mpc_score"}, edges, step_metadata=smd)
        walk = "prefill_video_encoder_only" if task == "encode" else "prefill_video"
        return ForwardPassArgs({"graph_walk": walk}, edges, step_metadata=smd)

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        ts = [output] if isinstance(output, torch.Tensor) else list(output)
        return torch.cat([t.float().reshape(-1) for t in ts]).numpy().tobytes()


class VJepa2ACModel(VJepa2Model):
    name = "vjepa2_ac"
    action_conditioned = True
