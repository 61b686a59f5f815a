"""Pi0.5 class vision-language-action policy: SigLIP image tokens and the tokenised instruction / robot state form
a bidirectional prefix run through a PaliGemma-style decoder (K/V cached); a smaller "action expert" with the same
head geometry denoises a chunk of future actions in 10 flow-matching steps, attending to [cached prefix ‖ action
tokens]. The expert's norms are adaptive (adaRMS): scale, shift and a residual gate come from the flow time.

Walks: ``prefill`` (vit_encoder, then the bidirectional prefix), ``action_gen`` (Loop ``action_loop`` x 10).
Reference counterparts: mstar/model/pi05/pi05_model.py (728 lines), submodules.py (809), components/* (365),
adaptive RMSNorm kernel (mstar/utils/adarms_norm.py:31-77), image normalisation kernel
(mstar/model/pi05/kernels/image_normalize.py).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop, Sequential
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from .base import small_scale, EngineType, ForwardPassArgs, Model
from .encoders import EncoderConfig, VisionEncoder
from .submodule_base import ARNodeInputs, ARNodeSubmodule, NodeSubmodule


def _p(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


class GemmaTower(nn.Module):
    """Gemma-style decoder stack: (1 + w) RMSNorm, GeGLU MLP, rotary embedding. ``adaptive``: norms are modulated by
    a conditioning vector (dense -> scale, shift, gate) instead of a learned weight."""

    def __init__(self, hidden, layers, heads, kv_heads, head_dim, ffn, adaptive: bool, dtype, device, theta=10000.0):
        super().__init__()
        self.H, self.nh, self.nkv, self.D, self.adaptive, self.dtype = hidden, heads, kv_heads, head_dim, adaptive, dtype
        self.layers = nn.ModuleList()
        for _ in range(layers):
            L = nn.Module()
            L.qkv = _p(((heads + 2 * kv_heads) * head_dim, hidden), dtype, device)
            L.o = _p((hidden, heads * head_dim), dtype, device)
            L.gate_up = _p((2 * ffn, hidden), dtype, device)          # gate rows then up rows
            L.down = _p((hidden, ffn), dtype, device)
            if adaptive:
                L.mod1_w, L.mod1_b = _p((3 * hidden, hidden), dtype, device), _p((3 * hidden,), dtype, device)
                L.mod2_w, L.mod2_b = _p((3 * hidden, hidden), dtype, device), _p((3 * hidden,), dtype, device)
            else:
                L.n1, L.n2 = _p((hidden,), dtype, device), _p((hidden,), dtype, device)
            self.layers.append(L)
        if adaptive:
            self.modf_w, self.modf_b = _p((3 * hidden, hidden), dtype, device), _p((3 * hidden,), dtype, device)
        else:
            self.nf = _p((hidden,), dtype, device)
        self.inv_freq = rope_ops.make_inv_freq(head_dim, theta, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1])).to(p.dtype))
        return self

    def _norm(self, x, w, mod_w, mod_b, cond):
        """Returns (normed, gate or None)."""
        if not self.adaptive:
            return norm_ops.norm(x, w, 1e-6, gemma=True)[0], None
        m = gemm.linear(cond, mod_w, bias=mod_b).reshape(-1, 3, self.H)            # [n_cond, (scale, shift, gate), H]
        return norm_ops.norm(x, None, 1e-6, scale=m[:, 0], shift=m[:, 1])[0], m[:, 2]

    def layer(self, li, x, positions, attend, cond=None, cache_args=None):
        L = self.layers[li]
        h, gate = self._norm(x, getattr(L, "n1", None), getattr(L, "mod1_w", None), getattr(L, "mod1_b", None), cond)
        qkv = gemm.linear(h, L.qkv)
        q, k, v = rope_ops.rope_kv(qkv, positions, self.inv_freq, self.nh, self.nkv, self.D,
                                   dense_kv=cache_args is None, **(cache_args or {}))
        a = attend(li, q, k, v)
        y = gemm.linear(a.reshape(a.shape[0], -1), L.o)
        x = ew.gated_residual(x, y, gate)
        h, gate = self._norm(x, getattr(L, "n2", None), getattr(L, "mod2_w", None), getattr(L, "mod2_b", None), cond)
        y = gemm.linear(ew.act_mul(gemm.linear(h, L.gate_up), "gelu"), L.down)
        return ew.gated_residual(x, y, gate)

    def final(self, x, cond=None):
        if self.adaptive:
            return self._norm(x, None, self.modf_w, self.modf_b, cond)[0]
        return norm_ops.norm(x, self.nf, 1e-6, gemma=True)[0]


def flow_time_embedding(t: torch.Tensor, dim: int, min_period: float = 4e-3, max_period: float = 4.0) -> torch.Tensor:
    """fp32 [n, dim], sine half then cosine half, periods spaced geometrically from ``min_period`` to ``max_period``
    (computed in fp64: the short periods lose digits otherwise and the error compounds through the adaptive norms).
    Reference: mstar/model/pi05/components/flow_matching.py:7-42."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64, device=t.device)
    omega = 2.0 * math.pi / (min_period * (max_period / min_period) ** frac)
    ang = t.to(torch.float64).reshape(-1, 1) * omega
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1).float()


def state_bins(state, bins: int = 256) -> list[int]:
    """Robot state in [-1, 1] -> bin indices (mstar/model/pi05/components/flow_matching.py:53-75)."""
    s = torch.as_tensor(state, dtype=torch.float32).clamp(-1.0, 1.0)
    return ((s + 1.0) / 2.0 * (bins - 1)).round().long().clamp(0, bins - 1).tolist()


class Pi05Policy(nn.Module):
    def __init__(self, *, vocab, hidden, layers, heads, kv_heads, head_dim, ffn, a_hidden, a_ffn, action_dim, dtype, device):
        super().__init__()
        self.dtype, self.device, self.action_dim, self.H = dtype, torch.device(device), action_dim, hidden
        self.embed = _p((vocab, hidden), dtype, device)
        self.und = GemmaTower(hidden, layers, heads, kv_heads, head_dim, ffn, False, dtype, device)
        self.act = GemmaTower(a_hidden, layers, heads, kv_heads, head_dim, a_ffn, True, dtype, device)
        self.a_in_w, self.a_in_b = _p((a_hidden, action_dim), dtype, device), _p((a_hidden,), dtype, device)
        self.a_out_w, self.a_out_b = _p((action_dim, a_hidden), dtype, device), _p((action_dim,), dtype, device)
        self.t1_w, self.t1_b = _p((a_hidden, a_hidden), dtype, device), _p((a_hidden,), dtype, device)
        self.t2_w, self.t2_b = _p((a_hidden, a_hidden), dtype, device), _p((a_hidden,), dtype, device)

    def init_random(self, seed=0):
        self.und.init_random(seed)
        self.act.init_random(seed + 1)
        g = torch.Generator().manual_seed(seed + 2)
        for n, p in self.named_parameters():
            if not n.startswith(("und.", "act.")):
                p.data.copy_((torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 1 else 1 / math.sqrt(p.shape[-1]))).to(p.dtype))
        return self

    def prefix(self, x: torch.Tensor, ctx) -> None:
        """Bidirectional prefix: writes K/V of all rows, then every row attends to all of them."""
        pos = ctx.positions if ctx.positions.dim() == 1 else ctx.positions[0]
        for li in range(len(self.und.layers)):
            kv = ctx.kv(li)
            ca = dict(cache=kv, token_req=ctx.token_req, cache_pos=ctx.cache_pos, page_indptr=ctx.plan.page_indptr,
                      page_indices=ctx.plan.page_indices)
            x = self.und.layer(li, x, pos, lambda i, q, k, v, kv=kv: attn_ops.attention(q, ctx.plan, kv_cache=kv),
                               cache_args=ca)

    def action_velocity(self, actions: torch.Tensor, t: float, prefix_ctx, pos0: int) -> torch.Tensor:
        """actions: [horizon, action_dim] fp32 -> velocity, same shape (fp32)."""
        n = actions.shape[0]
        x = gemm.linear(actions.to(self.dtype), self.a_in_w, bias=self.a_in_b)
        e = flow_time_embedding(torch.tensor([t], device=x.device), x.shape[-1]).to(self.dtype)
        c = gemm.linear(e, self.t1_w, bias=self.t1_b)
        c = gemm.linear(torch.nn.functional.silu(c.float()).to(c.dtype), self.t2_w, bias=self.t2_b)
        cond = torch.nn.functional.silu(c.float()).to(c.dtype)                      # [1, a_hidden]
        pos = torch.arange(n, dtype=torch.int32, device=x.device) + pos0
        G = max(1, self.act.nh // self.act.nkv)
        plan = attn_ops.dense_plan([n], [n], G, x.device, causal=False)

        def attend(li, q, k, v):
            o_f, l_f = attn_ops.attention(q, plan, k=k, v=v, lse=True)
            o_p, l_p = attn_ops.attention(q, prefix_ctx.plan, kv_cache=prefix_ctx.kv(li), lse=True)
            return attn_ops.attn_merge(o_p, l_p, o_f, l_f)
        for li in range(len(self.act.layers)):
            x = self.act.layer(li, x, pos, attend, cond=cond)
        return gemm.linear(self.act.final(x, cond), self.a_out_w, bias=self.a_out_b, out_dtype=torch.float32)


class Pi05VitSubmodule(NodeSubmodule):
    """Normalises camera frames to [-1, 1] (fused affine kernel on the GPU) and encodes them."""

    def __init__(self, enc: VisionEncoder, device):
        super().__init__(device, enc.c.dtype)
        self.enc = enc

    def forward(self, graph_walk, engine_inputs, ni, **kw):
        imgs = []
        for t in ni.tensor_inputs["image"]:
            t = t.to(self.device).float()
            imgs.append(ew.affine(t.contiguous(), 2.0, -1.0, out_dtype=self.dtype) if t.min() >= 0 else t.to(self.dtype))
        feats, _, _ = self.enc(imgs)
        return {"image_features": feats}


class Pi05LLMSubmodule(ARNodeSubmodule):
    IMG = 257152 - 1

    def __init__(self, m: Pi05Policy, device, horizon: int, steps: int):
        super().__init__(device, m.dtype)
        self.m, self.horizon, self.steps = m, horizon, steps

    def prepare_inputs(self, graph_walk, fwd_info, inputs):
        ni = ARNodeInputs(fwd_info.request_id, graph_walk, inputs, dict(fwd_info.step_metadata or {}))
        if graph_walk == "prefill":
            n_img = sum(t.reshape(-1, t.shape[-1]).shape[0] for t in inputs.get("image_features", []))
            ids = torch.cat([t.reshape(-1) for t in inputs["input_ids"]]).to(torch.int64)
            ni.input_ids, ni.input_seq_len = ids, n_img + int(ids.numel())
        return ni

    def custom_plan(self, cache, graph_walk, prepared):
        ni = prepared.node_inputs[0]
        G = max(1, self.m.und.nh // self.m.und.nkv)
        if graph_walk == "prefill":
            return cache.plan([ni.request_id], [ni.input_seq_len], causal=False, group=G)
        return cache.plan([ni.request_id], [self.horizon], causal=False, write_cache=False, group=G)

    def can_batch(self, graph_walk):
        return False

    def max_batch_size(self, graph_walk):
        return 1

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ni, ctx, m = inputs[0], engine_inputs.batch_context, self.m
        st = engine_inputs.per_request_states[ni.request_id]
        if graph_walk == "prefill":
            # the published weights expect image tokens scaled by sqrt(H) and text rows by H (the checkpoint's own
            # embedding layer scales by sqrt(H) once and the policy's prefix builder a second time:
            # mstar/model/pi05/submodules.py:306-326)
            parts = [ew.affine(t.reshape(-1, m.H).to(self.device, m.dtype).contiguous(), math.sqrt(m.H), 0.0, out_dtype=m.dtype)
                     for t in ni.tensor_inputs.get("image_features", [])]
            parts.append(ew.embed(ni.input_ids.to(self.device), m.embed, scale=float(m.H)))
            m.prefix(torch.cat(parts).contiguous(), ctx)
            st["prefix_len"] = ni.input_seq_len
            return [{"prefill_done": torch.tensor([ni.input_seq_len], dtype=torch.int64)}]
        if ni.tensor_inputs.get("actions"):
            x = ni.tensor_inputs["actions"][-1].to(self.device, torch.float32)
        else:
            info = engine_inputs.per_request_info[ni.request_id]
            g = torch.Generator().manual_seed(int(ni.kwargs.get("seed", info.random_seed or 0)))
            x = torch.randn((self.horizon, m.action_dim), generator=g).to(self.device)
            st["i"] = 0
        n = int(ni.kwargs.get("num_steps", self.steps))
        t = 1.0 - st["i"] / n                          # time runs from noise (1) to data (0)
        st["i"] += 1
        v = m.action_velocity(x, t, ctx, int(st.get("prefix_len", 0)))
        return [{"actions": x - v / n}]

    def postprocess(self, request_id, request_info, outputs, inputs):
        return {k: v for k, v in outputs.items() if k not in ("new_token", "new_token_host")}


class Pi05Model(Model):
    name = "pi05"

    def __init__(self, model_dir=None, skip_weight_loading=False, small: bool = False, action_horizon: int = 50,
                 action_dim: int = 32, num_steps: int = 10, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self.small, self.dtype, self.horizon, self.action_dim, self.num_steps = small, dt, action_horizon, action_dim, num_steps
        if small:
            k = small_scale()
            self.kw = dict(vocab=1024, hidden=64 * k, layers=2, heads=4, kv_heads=1, head_dim=16 * k, ffn=128 * k,
                           a_hidden=32 * k, a_ffn=64 * k)
            self.vit_cfg, self.patch = EncoderConfig(32 * k, 1, 2, 16 * k, 64 * k, dtype=dt), 4
            self.horizon = min(self.horizon, 8)
        else:
            self.kw = dict(vocab=257152, hidden=2048, layers=18, heads=8, kv_heads=1, head_dim=256, ffn=16384,
                           a_hidden=1024, a_ffn=4096)
            self.vit_cfg, self.patch = EncoderConfig(1152, 27, 16, 72, 4304, dtype=dt), 14

    def get_graph_walk_graphs(self):
        vit = GraphNode("vit_encoder", {"image"}, [GraphEdge("LLM", "image_features")])
        pre = GraphNode("LLM", {"input_ids", "image_features"}, [GraphEdge(EMPTY_DESTINATION, "prefill_done", persist=True)])
        step = GraphNode("LLM", {"actions"}, [GraphEdge("LLM", "actions")], enable_async_scheduling=False)
        return {"prefill": Sequential([vit, pre]),
                "action_gen": Loop(step, max_iters=self.num_steps, name="action_loop",
                                   outputs=[GraphEdge(EMIT_TO_CLIENT, "actions", output_modality="action")])}

    def get_node_engine_types(self):
        return {"vit_encoder": EngineType.STATELESS, "LLM": EngineType.KV_CACHE}

    def get_kv_cache_config(self):
        k = self.kw
        return [KVCacheConfig(k["layers"], k["kv_heads"], k["head_dim"], max_seq_len=4096,
                              max_num_pages=32 if self.small else 256, page_size=16 if self.small else 128,
                              num_qo_heads=k["heads"], nodes=["LLM"], dtype=self.dtype)]

    def get_engine_hints(self, node):
        return dict(vocab_size=8, group=self.kw["heads"] // self.kw["kv_heads"], max_tokens=4096, track_seen=False,
                    max_batch=16)

    def get_autocast_dtype(self):
        return self.dtype

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        if node_name == "vit_encoder":
            enc = VisionEncoder(self.vit_cfg, patch=self.patch, pos="learned", pos_grid=4 if self.small else 16,
                                out_dim=self.kw["hidden"], device=device, projector="linear").init_random(0)
            if not (self.skip_weight_loading or self.model_dir is None):
                from .checkpoints import load_pi05_vision
                load_pi05_vision(enc, self._checkpoint())
            return Pi05VitSubmodule(enc, device)
        if node_name == "LLM":
            m = Pi05Policy(action_dim=self.action_dim, dtype=self.dtype, device=device, **self.kw).init_random(0)
            if not (self.skip_weight_loading or self.model_dir is None):
                from .checkpoints import load_pi05_policy
                load_pi05_policy(m, self._checkpoint())
            return Pi05LLMSubmodule(m, device, self.horizon, self.num_steps)
        raise KeyError(node_name)

    def _checkpoint(self) -> str:
        """The published policy is one ``model.safetensors`` in the snapshot directory."""
        import os
        one = os.path.join(self.model_dir, "model.safetensors")
        return one if os.path.exists(one) else self.model_dir

    MAX_LANG_TOKENS = 200

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, state: list | None = None,
                       robot_state: list | None = None, **kw):
        v = self.kw["vocab"]
        state = state if state is not None else robot_state
        if self.tokenizer() is not None:
            # the published prompt format: lower-cased task, the state's bin indices as text
            # (mstar/model/pi05/pi05_model.py:470-505, components/tokenization.py:12-34)
            text = (prompt or "").strip().replace("_", " ").replace("\n", " ")
            if state is not None and len(state):
                text = f"Task: {text}, State: {' '.join(str(b) for b in state_bins(state))};\nAction: "
            ids = list(self.tokenizer()(text.strip().lower(), add_special_tokens=True).input_ids)[:self.MAX_LANG_TOKENS]
        else:
            ids = self.encode_text(prompt, v, v - 300, default="do the task")
            if state is not None and len(state):        # without a tokenizer: one reserved id per state bin
                ids += [v - 300 + b for b in state_bins(state)]
        if not tensors.get("image"):
            raise ValueError("the policy needs at least one camera image")
        return {"input_ids": [torch.tensor(ids, dtype=torch.int64)], "image": [t.float() for t in tensors["image"]]}

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        return ForwardPassArgs({"graph_walk": "prefill"},
                               [GraphEdge("LLM", "input_ids", list(input_signals["input_ids"])),
                                GraphEdge("vit_encoder", "image", list(input_signals["image"]))])

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        md = partition_metadata
        mk = md.get("model_kwargs") or {}
        if md["finished_walk"] == "prefill":
            n = int(mk.get("num_steps", self.num_steps))
            return ForwardPassArgs({"graph_walk": "action_gen", "dynamic_loop_iter_counts": {"action_loop": n}},
                                   [GraphEdge("LLM", "actions", [])],
                                   step_metadata={"num_steps": n, **({"seed": mk["seed"]} if "seed" in mk else {})})
        return ForwardPassArgs(request_done=True)

    def postprocess(self, output, modality, request_kwargs):
        t = output if isinstance(output, torch.Tensor) else output[-1]
        return t.float().contiguous().numpy().tobytes()


class Pi05DroidModel(Pi05Model):
    """DROID robot platform variant: 15-step action chunks of 8 dimensions."""
    name = "pi05_droid"

    def __init__(self, *a, **kw):
        kw.setdefault("action_horizon", 15)
        kw.setdefault("action_dim", 8)
        super().__init__(*a, **kw)
