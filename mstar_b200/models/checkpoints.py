"""Loaders for the checkpoint layouts that the served models are published in (Hugging Face / diffusers tensor
names), into this library's fused parameters. Every loader is STRICT: a checkpoint tensor that reaches no
parameter, a parameter that no tensor reached, or a shape that does not fit raises ``CheckpointMismatch`` — a
silently skipped weight is a wrong-output bug, not a warning.

  * ``load_wan22_transformer``   diffusers ``WanTransformer3DModel`` (``transformer/diffusion_pytorch_model*``):
                                 q/k/v rows stacked into ``qkv_w``, the cross-attention k/v into ``ckv_w``, the
                                 Conv3d patch embedding flattened to a GEMM weight, scale-shift tables kept fp32.
  * ``load_whisper``             Hugging Face ``WhisperForConditionalGeneration`` names.
  * ``load_t5_encoder``          Hugging Face ``UMT5EncoderModel`` / ``T5EncoderModel`` names.
  * ``load_siglip_vision``, ``load_bagel_mot``, ``load_image_autoencoder``   the three files of a published BAGEL
                                 checkpoint (vision tower, both experts, latent autoencoder).

Reference counterparts: mstar/model/wan22/weight_loader.py:34-138 (key remap and completeness contract),
mstar/model/cosmos3/loader.py:25-126, mstar/model/loader/base.py (stacked-parameter rules).
"""
from __future__ import annotations

import json
import os
from collections.abc import Iterator

import torch


class CheckpointMismatch(RuntimeError):
    pass


def iter_checkpoint(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, CPU tensor) for every tensor under ``path``: a directory with a transformers or diffusers index file,
    a directory of ``*.safetensors`` files, or one safetensors file."""
    from safetensors import safe_open
    if os.path.isfile(path):
        files, base = [os.path.basename(path)], os.path.dirname(path)
    else:
        base, files = path, []
        for idx in ("model.safetensors.index.json", "diffusion_pytorch_model.safetensors.index.json"):
            p = os.path.join(path, idx)
            if os.path.exists(p):
                with open(p) as f:
                    files = sorted(set(json.load(f)["weight_map"].values()))
                break
        if not files:
            files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors checkpoint in {path}")
    for fn in files:
        with safe_open(os.path.join(base, fn), framework="pt", device="cpu") as f:
            for k in f.keys():
                yield k, f.get_tensor(k)


class _Filler:
    """Bookkeeping of a strict load: which parameters were written (whole or by row ranges), which checkpoint keys
    found no home."""

    def __init__(self, module: torch.nn.Module, what: str):
        self.params = dict(module.named_parameters())
        self.params.update(dict(module.named_buffers()))
        self.what = what
        self.filled: dict[str, int] = {}          # parameter -> rows written
        self.unexpected: list[str] = []
        self.bad_shape: list[str] = []

    @torch.no_grad()
    def put(self, key: str, name: str, t: torch.Tensor, rows: tuple[int, int] | None = None) -> None:
        p = self.params.get(name)
        if p is None:
            self.unexpected.append(key)
            return
        dst = p if rows is None else p[rows[0]:rows[1]]
        if tuple(dst.shape) != tuple(t.shape):
            if dst.numel() == t.numel() and rows is None:
                t = t.reshape(dst.shape)           # Conv3d patch embedding -> GEMM weight, [1, n, H] tables -> [n, H]
            else:
                self.bad_shape.append(f"{key} {tuple(t.shape)} -> {name} {tuple(dst.shape)}")
                return
        dst.copy_(t.to(dst.dtype))
        self.filled[name] = self.filled.get(name, 0) + (dst.shape[0] if dst.dim() else 1)

    def finish(self, ignore: tuple[str, ...] = ()) -> dict:
        missing = []
        for name, p in self.params.items():
            if any(name.startswith(i) for i in ignore):
                continue
            want = p.shape[0] if p.dim() else 1
            if self.filled.get(name, 0) != want:
                missing.append(f"{name} ({self.filled.get(name, 0)}/{want} rows)")
        if self.unexpected or missing or self.bad_shape:
            raise CheckpointMismatch(
                f"{self.what}: {len(self.unexpected)} checkpoint keys without a parameter {self.unexpected[:5]}, "
                f"{len(missing)} parameters not (fully) loaded {missing[:5]}, {len(self.bad_shape)} shape mismatches "
                f"{self.bad_shape[:5]}")
        return {"loaded": len(self.filled)}


# ------------------------------------------------------------------ Wan2.2 (diffusers WanTransformer3DModel)
_WAN_TOP = {
    "patch_embedding.weight": "patch_w", "patch_embedding.bias": "patch_b",
    "condition_embedder.text_embedder.linear_1.weight": "text1_w", "condition_embedder.text_embedder.linear_1.bias": "text1_b",
    "condition_embedder.text_embedder.linear_2.weight": "text2_w", "condition_embedder.text_embedder.linear_2.bias": "text2_b",
    "condition_embedder.time_embedder.linear_1.weight": "time1_w", "condition_embedder.time_embedder.linear_1.bias": "time1_b",
    "condition_embedder.time_embedder.linear_2.weight": "time2_w", "condition_embedder.time_embedder.linear_2.bias": "time2_b",
    "condition_embedder.time_proj.weight": "tproj_w", "condition_embedder.time_proj.bias": "tproj_b",
    "scale_shift_table": "head_mod", "proj_out.weight": "head_w", "proj_out.bias": "head_b",
}
_WAN_BLOCK = {
    "scale_shift_table": ("modulation", None),
    "attn1.to_q.weight": ("qkv_w", 0), "attn1.to_k.weight": ("qkv_w", 1), "attn1.to_v.weight": ("qkv_w", 2),
    "attn1.to_q.bias": ("qkv_b", 0), "attn1.to_k.bias": ("qkv_b", 1), "attn1.to_v.bias": ("qkv_b", 2),
    "attn1.norm_q.weight": ("norm_q", None), "attn1.norm_k.weight": ("norm_k", None),
    "attn1.to_out.0.weight": ("o_w", None), "attn1.to_out.0.bias": ("o_b", None),
    "norm2.weight": ("norm3_w", None), "norm2.bias": ("norm3_b", None),
    "attn2.to_q.weight": ("cq_w", None), "attn2.to_q.bias": ("cq_b", None),
    "attn2.to_k.weight": ("ckv_w", 0), "attn2.to_v.weight": ("ckv_w", 1),
    "attn2.to_k.bias": ("ckv_b", 0), "attn2.to_v.bias": ("ckv_b", 1),
    "attn2.norm_q.weight": ("cnorm_q", None), "attn2.norm_k.weight": ("cnorm_k", None),
    "attn2.to_out.0.weight": ("co_w", None), "attn2.to_out.0.bias": ("co_b", None),
    "ffn.net.0.proj.weight": ("ffn1_w", None), "ffn.net.0.proj.bias": ("ffn1_b", None),
    "ffn.net.2.weight": ("ffn2_w", None), "ffn.net.2.bias": ("ffn2_b", None),
}


@torch.no_grad()
def load_wan22_transformer(dit, transformer_dir: str) -> dict:
    """Fill an ``AdaLNDiT`` from a diffusers Wan2.2 transformer directory (or file). A tensor-parallel model is
    filled through a full-size copy on the host (strict there), of which every rank keeps its heads and MLP columns."""
    if getattr(dit, "tp", None) is not None and dit.tp.size > 1:      # (sequence-parallel ranks hold whole weights)
        from .dit import AdaLNDiT, adaln_shard
        full = AdaLNDiT(dit.cfg, "cpu")
        info = load_wan22_transformer(full, transformer_dir)
        src = dict(full.named_parameters())
        for n, p in dit.named_parameters():
            p.copy_(adaln_shard(n, src[n], dit.tp.rank, dit.tp.size).to(p.dtype))
        return info
    H = dit.cfg.hidden_size
    fill = _Filler(dit, f"Wan2.2 transformer at {transformer_dir}")
    for key, t in iter_checkpoint(transformer_dir):
        if key in _WAN_TOP:
            fill.put(key, _WAN_TOP[key], t)
            continue
        parts = key.split(".", 2)
        if len(parts) == 3 and parts[0] == "blocks" and parts[1].isdigit() and parts[2] in _WAN_BLOCK:
            name, slot = _WAN_BLOCK[parts[2]]
            full = f"blocks.{parts[1]}.{name}"
            fill.put(key, full, t, None if slot is None else (slot * H, (slot + 1) * H))
        else:
            fill.unexpected.append(key)
    return fill.finish()


def wan22_checkpoint_keys(dit) -> dict[str, torch.Tensor]:
    """The inverse of ``load_wan22_transformer``: this module's weights under the diffusers tensor names (used to
    write checkpoints, e.g. synthetic ones for tests and benchmarks)."""
    cfg, H = dit.cfg, dit.cfg.hidden_size
    sd = {n: p.detach() for n, p in dit.named_parameters()}
    out = {}
    for k, n in _WAN_TOP.items():
        t = sd[n]
        if k == "patch_embedding.weight":
            t = t.reshape(H, cfg.in_channels, *cfg.patch_size)
        elif k == "scale_shift_table":
            t = t.reshape(1, 2, H)
        out[k] = t.contiguous()
    for i in range(cfg.num_layers):
        for k, (n, slot) in _WAN_BLOCK.items():
            t = sd[f"blocks.{i}.{n}"]
            if slot is not None:
                t = t[slot * H:(slot + 1) * H]
            elif k == "scale_shift_table":
                t = t.reshape(1, 6, H)
            out[f"blocks.{i}.{k}"] = t.contiguous()
    return out


# ------------------------------------------------------------------ Cosmos3 (diffusers dual-pathway transformer)
_C3_TOP = {
    "proj_in.weight": "proj_in_w", "proj_in.bias": "proj_in_b", "proj_out.weight": "proj_out_w", "proj_out.bias": "proj_out_b",
    "time_embedder.linear_1.weight": "t1_w", "time_embedder.linear_1.bias": "t1_b",
    "time_embedder.linear_2.weight": "t2_w", "time_embedder.linear_2.bias": "t2_b",
    "audio_proj_in.weight": "audio_in_w", "audio_proj_in.bias": "audio_in_b",
    "audio_proj_out.weight": "audio_out_w", "audio_proj_out.bias": "audio_out_b",
    "audio_modality_embed": "audio_modality_embed", "action_modality_embed": "action_modality_embed",
    "action_proj_in.fc.weight": "act_in_fc", "action_proj_in.bias.weight": "act_in_bias",
    "action_proj_out.fc.weight": "act_out_fc", "action_proj_out.bias.weight": "act_out_bias",
    "norm.weight": "und.norm", "norm_moe_gen.weight": "gen.final_norm",
}
_C3_DROP = ("lm_head.weight",)           # the understanding tower descends from a text model; its head is never used
# per layer: checkpoint suffix -> (tower, parameter, role)
_C3_LAYER = {
    "input_layernorm.weight": ("und", "input_layernorm", None),
    "post_attention_layernorm.weight": ("und", "post_attention_layernorm", None),
    "input_layernorm_moe_gen.weight": ("gen", "input_norm", None),
    "post_attention_layernorm_moe_gen.weight": ("gen", "post_norm", None),
    "self_attn.norm_q.weight": ("und", "self_attn.q_norm", None), "self_attn.norm_k.weight": ("und", "self_attn.k_norm", None),
    "self_attn.norm_added_q.weight": ("gen", "q_norm", None), "self_attn.norm_added_k.weight": ("gen", "k_norm", None),
    "self_attn.to_q.weight": ("und", "qkv", "q"), "self_attn.to_k.weight": ("und", "qkv", "k"),
    "self_attn.to_v.weight": ("und", "qkv", "v"), "self_attn.to_out.weight": ("und", "o", None),
    "self_attn.add_q_proj.weight": ("gen", "qkv", "q"), "self_attn.add_k_proj.weight": ("gen", "qkv", "k"),
    "self_attn.add_v_proj.weight": ("gen", "qkv", "v"), "self_attn.to_add_out.weight": ("gen", "o", None),
    "mlp.gate_proj.weight": ("und", "mlp", "gate"), "mlp.up_proj.weight": ("und", "mlp", "up"),
    "mlp.down_proj.weight": ("und", "mlp", "down"),
    "mlp_moe_gen.gate_proj.weight": ("gen", "mlp", "gate"), "mlp_moe_gen.up_proj.weight": ("gen", "mlp", "up"),
    "mlp_moe_gen.down_proj.weight": ("gen", "mlp", "down"),
}


@torch.no_grad()
def load_cosmos3_transformer(m, transformer_dir: str) -> dict:
    """Fill a ``Cosmos3Transformer`` (any tensor- / sequence-parallel cut) from the published ``transformer/``
    layout: flat ``layers.N.*`` keys, unfused ``to_q / to_k / to_v`` for the understanding pathway and
    ``add_q_proj / add_k_proj / add_v_proj`` for the generation pathway, ``*_moe_gen`` MLPs and norms of the generation
    pathway, domain tables of the action projections. q / k / v become the rows of one fused projection per pathway
    (this rank's heads), gate and up the interleaved rows of one projection whose epilogue applies SwiGLU. Strict:
    every parameter must be reached, every key must have a home (except the unused text head)."""
    import re
    from ..ops import gemm
    from .decoder import shard_qkv
    cfg = m.cfg
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    params = dict(m.named_parameters())
    filled: set[str] = set()
    unexpected: list[str] = []
    bad: list[str] = []
    groups: dict[tuple, dict] = {}
    rx = re.compile(r"layers\.(\d+)\.(.+)")

    def put(name: str, t: torch.Tensor, key: str):
        p = params.get(name)
        if p is None:
            unexpected.append(key)
        elif tuple(p.shape) != tuple(t.shape):
            bad.append(f"{key} {tuple(t.shape)} -> {name} {tuple(p.shape)}")
        else:
            p.copy_(t.to(p.dtype))
            filled.add(name)

    def tower(which: str):
        """(module path prefix of layer li, tensor-parallel group, attention module path, mlp module path)."""
        if which == "und":
            return m.und.tp, (lambda li: f"und.layers.{li}."), "self_attn.", "mlp."
        return m.gen.tp, (lambda li: f"gen.layers.{li}."), "", ""

    for key, t in iter_checkpoint(transformer_dir):
        if key in _C3_DROP:
            continue
        if key == "embed_tokens.weight":
            put("und.embed_tokens", m.und.vocab_rows(t) if hasattr(m.und, "vocab_rows") else t, key)
            continue
        if key in _C3_TOP:
            put(_C3_TOP[key], t, key)
            continue
        mt = rx.fullmatch(key)
        if not mt or mt.group(2) not in _C3_LAYER or int(mt.group(1)) >= cfg.num_layers:
            unexpected.append(key)
            continue
        li, (tw, what, role) = int(mt.group(1)), _C3_LAYER[mt.group(2)]
        tp, lpre, apre, mpre = tower(tw)
        if role is None and what != "o":
            put(lpre(li) + what, t, key)
        elif what == "o":
            hq = Hq // tp.size
            put(lpre(li) + apre + "o_proj", t[:, tp.rank * hq * D:(tp.rank + 1) * hq * D], key)
        else:
            g = groups.setdefault((tw, li, what), {})
            g[role] = (t, key)
            need = ("q", "k", "v") if what == "qkv" else ("gate", "up", "down")
            if all(r in g for r in need):
                if what == "qkv":
                    fused = shard_qkv(g["q"][0], g["k"][0], g["v"][0], Hq, Hkv, D, tp.rank, tp.size)
                    put(lpre(li) + apre + "qkv_proj", fused, g["q"][1])
                else:
                    F = g["gate"][0].shape[0] // tp.size
                    sl = slice(tp.rank * F, (tp.rank + 1) * F)
                    put(lpre(li) + mpre + "gate_up_proj", gemm.interleave_gate_up(g["gate"][0][sl], g["up"][0][sl]), g["gate"][1])
                    put(lpre(li) + mpre + "down_proj", g["down"][0][:, sl], g["down"][1])
                del groups[(tw, li, what)]
    incomplete = [f"{tw}.layers.{li}.{what}: only {sorted(g)}" for (tw, li, what), g in groups.items()]
    missing = sorted(set(params) - filled)
    if unexpected or missing or bad or incomplete:
        raise CheckpointMismatch(
            f"Cosmos3 transformer: {len(unexpected)} checkpoint keys without a parameter {unexpected[:5]}, "
            f"{len(missing)} parameters not loaded {missing[:5]}, {len(bad)} shape mismatches {bad[:5]}, "
            f"{len(incomplete)} incomplete projection groups {incomplete[:3]}")
    m._domain_w.clear()
    return {"loaded": len(filled)}


def cosmos3_checkpoint_keys(m) -> dict[str, torch.Tensor]:
    """The published key layout of an (unsharded) ``Cosmos3Transformer``'s weights: the inverse of the loader, for
    synthetic checkpoints in tests and for export."""
    from ..ops import gemm
    cfg = m.cfg
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    sd = {k: v.detach().clone() for k, v in m.named_parameters()}
    out = {ck: sd[name] for ck, name in _C3_TOP.items()}
    out["embed_tokens.weight"] = sd["und.embed_tokens"]
    for li in range(cfg.num_layers):
        for suffix, (tw, what, role) in _C3_LAYER.items():
            pre = f"und.layers.{li}." if tw == "und" else f"gen.layers.{li}."
            apre, mpre = ("self_attn.", "mlp.") if tw == "und" else ("", "")
            key = f"layers.{li}.{suffix}"
            if role is None and what != "o":
                out[key] = sd[pre + what]
            elif what == "o":
                out[key] = sd[pre + apre + "o_proj"]
            elif what == "qkv":
                w = sd[pre + apre + "qkv_proj"]
                q, k, v = w[:Hq * D], w[Hq * D:(Hq + Hkv) * D], w[(Hq + Hkv) * D:]
                out[key] = {"q": q, "k": k, "v": v}[role].clone()
            else:
                if role == "down":
                    out[key] = sd[pre + mpre + "down_proj"]
                else:
                    gate, up = gemm.split_gate_up(sd[pre + mpre + "gate_up_proj"])
                    out[key] = (gate if role == "gate" else up).clone()
    return out


# ------------------------------------------------------------------ helpers for the Hugging Face encoder layouts
def _tensors_of(src) -> dict[str, torch.Tensor]:
    return dict(src) if isinstance(src, dict) else dict(iter_checkpoint(src))


class _Strict:
    """Copy checkpoint tensors into parameters and account for both sides: ``done()`` raises unless every parameter
    was written and every checkpoint key was taken (or explicitly ignored)."""

    def __init__(self, module: torch.nn.Module, tensors: dict[str, torch.Tensor], what: str):
        self.params = dict(module.named_parameters())
        self.tensors, self.what = tensors, what
        self.written: set[str] = set()
        self.taken: set[str] = set()
        self.bad: list[str] = []

    def take(self, key: str, optional: bool = False) -> torch.Tensor | None:
        t = self.tensors.get(key)
        if t is None:
            if not optional:
                self.bad.append(f"missing {key}")
            return None
        self.taken.add(key)
        return t

    @torch.no_grad()
    def write(self, name: str, t: torch.Tensor | None) -> None:
        p = self.params.get(name)
        if t is None or p is None:
            if p is None:
                self.bad.append(f"no parameter {name}")
            return
        if tuple(p.shape) != tuple(t.shape):
            self.bad.append(f"{name}: checkpoint {tuple(t.shape)} vs parameter {tuple(p.shape)}")
            return
        p.copy_(t.to(p.dtype))
        self.written.add(name)

    def done(self, ignore_keys=(), ignore_params=()) -> dict:
        left = sorted(k for k in set(self.tensors) - self.taken if not any(k.startswith(i) or k == i for i in ignore_keys))
        missing = sorted(n for n in set(self.params) - self.written if not any(n.startswith(i) for i in ignore_params))
        if left or missing or self.bad:
            raise CheckpointMismatch(f"{self.what}: {len(left)} checkpoint keys without a parameter {left[:5]}, "
                                     f"{len(missing)} parameters not loaded {missing[:5]}, problems {self.bad[:5]}")
        return {"loaded": len(self.written)}


def _cat_bias(parts: list[torch.Tensor | None], like: list[torch.Tensor]) -> torch.Tensor:
    """Fused bias of stacked projections; a projection without a bias (Whisper's key projection) contributes zeros."""
    return torch.cat([b if b is not None else torch.zeros(w.shape[0], dtype=w.dtype) for b, w in zip(parts, like)])


# ------------------------------------------------------------------ T5 / UMT5 encoder (Hugging Face names)
@torch.no_grad()
def load_t5_encoder(enc, src) -> dict:
    """``T5Encoder`` from a Hugging Face ``T5EncoderModel`` / ``UMT5EncoderModel`` checkpoint (directory or name ->
    tensor dict): q / k / v stacked into one projection, ``wi_0`` (gate) and ``wi_1`` (up) interleaved by rows, the
    relative-position table of every block (UMT5) or of block 0 only (T5)."""
    from ..ops import gemm
    T = _tensors_of(src)
    st = _Strict(enc, T, "T5 encoder")
    emb = st.take("shared.weight", optional=True)
    alt = st.take("encoder.embed_tokens.weight", optional=True)
    st.write("embed", emb if emb is not None else alt)
    if emb is None and alt is None:
        st.bad.append("missing shared.weight / encoder.embed_tokens.weight")
    L = len(enc.enc.layers)
    tables = []
    for i in range(L):
        a, f = f"encoder.block.{i}.layer.0.", f"encoder.block.{i}.layer.1."
        q, k, v = (st.take(a + f"SelfAttention.{n}.weight") for n in "qkv")
        if None not in (q, k, v):
            st.write(f"enc.layers.{i}.qkv_w", torch.cat([q, k, v]))
        st.write(f"enc.layers.{i}.o_w", st.take(a + "SelfAttention.o.weight"))
        st.write(f"enc.layers.{i}.n1_w", st.take(a + "layer_norm.weight"))
        g, u = st.take(f + "DenseReluDense.wi_0.weight"), st.take(f + "DenseReluDense.wi_1.weight")
        if g is not None and u is not None:
            st.write(f"enc.layers.{i}.fc1_w", gemm.interleave_gate_up(g, u))
        st.write(f"enc.layers.{i}.fc2_w", st.take(f + "DenseReluDense.wo.weight"))
        st.write(f"enc.layers.{i}.n2_w", st.take(f + "layer_norm.weight"))
        tb = st.take(a + "SelfAttention.relative_attention_bias.weight", optional=i > 0 or enc.rel_bias.shape[0] > 1)
        if tb is not None:
            tables.append(tb)
    if len(tables) == enc.rel_bias.shape[0]:
        st.write("rel_bias", torch.stack(tables))
    else:
        st.bad.append(f"{len(tables)} relative-position tables for {enc.rel_bias.shape[0]} expected")
    st.write("enc.fn_w", st.take("encoder.final_layer_norm.weight"))
    return st.done()


# ------------------------------------------------------------------ Whisper (Hugging Face names)
def _whisper_attn(st: _Strict, src: str, dst_w: str, dst_b: str, names=("q_proj", "k_proj", "v_proj")) -> None:
    ws = [st.take(f"{src}{n}.weight") for n in names]
    bs = [st.take(f"{src}{n}.bias", optional=n == "k_proj") for n in names]      # only the key projection has none
    if None not in ws:
        st.write(dst_w, torch.cat(ws))
        st.write(dst_b, _cat_bias(bs, ws))


@torch.no_grad()
def load_whisper_encoder(enc, src, prefix: str = "model.encoder.") -> dict:
    """``AudioEncoder`` from the encoder half of a Hugging Face Whisper checkpoint. Keys outside ``prefix`` are
    left alone (the decoder loads them)."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(enc, T, "Whisper encoder")
    for n in ("conv1", "conv2"):
        st.write(f"{n}.weight", st.take(f"{n}.weight"))
        st.write(f"{n}.bias", st.take(f"{n}.bias"))
    pos = st.take("embed_positions.weight")
    if pos is not None:
        if tuple(pos.shape) != tuple(enc.pos.shape):
            st.bad.append(f"embed_positions {tuple(pos.shape)} vs {tuple(enc.pos.shape)}")
        else:
            enc.pos.copy_(pos.to(enc.pos.dtype))
    for i in range(len(enc.enc.layers)):
        p, d = f"layers.{i}.", f"enc.layers.{i}."
        _whisper_attn(st, p + "self_attn.", d + "qkv_w", d + "qkv_b")
        st.write(d + "o_w", st.take(p + "self_attn.out_proj.weight"))
        st.write(d + "o_b", st.take(p + "self_attn.out_proj.bias"))
        for hf, ours in (("self_attn_layer_norm", "n1"), ("final_layer_norm", "n2")):
            st.write(d + ours + "_w", st.take(p + hf + ".weight"))
            st.write(d + ours + "_b", st.take(p + hf + ".bias"))
        for hf, ours in (("fc1", "fc1"), ("fc2", "fc2")):
            st.write(d + ours + "_w", st.take(p + hf + ".weight"))
            st.write(d + ours + "_b", st.take(p + hf + ".bias"))
    st.write("enc.fn_w", st.take("layer_norm.weight"))
    st.write("enc.fn_b", st.take("layer_norm.bias"))
    return st.done()


@torch.no_grad()
def load_whisper_decoder(dec, src, prefix: str = "model.decoder.") -> dict:
    """``WhisperDecoder`` from the decoder half of a Hugging Face Whisper checkpoint (the output head is the token
    embedding, as in the checkpoint; a separate ``proj_out.weight`` is accepted when it equals it)."""
    full = _tensors_of(src)
    T = {k[len(prefix):]: v for k, v in full.items() if k.startswith(prefix)}
    st = _Strict(dec, T, "Whisper decoder")
    st.write("tok", st.take("embed_tokens.weight"))
    st.write("pos", st.take("embed_positions.weight"))
    for i in range(len(dec.layers)):
        p, d = f"layers.{i}.", f"layers.{i}."
        _whisper_attn(st, p + "self_attn.", d + "qkv_w", d + "qkv_b")
        st.write(d + "o_w", st.take(p + "self_attn.out_proj.weight"))
        st.write(d + "o_b", st.take(p + "self_attn.out_proj.bias"))
        st.write(d + "cq_w", st.take(p + "encoder_attn.q_proj.weight"))
        st.write(d + "cq_b", st.take(p + "encoder_attn.q_proj.bias"))
        _whisper_attn(st, p + "encoder_attn.", d + "ckv_w", d + "ckv_b", names=("k_proj", "v_proj"))
        st.write(d + "co_w", st.take(p + "encoder_attn.out_proj.weight"))
        st.write(d + "co_b", st.take(p + "encoder_attn.out_proj.bias"))
        for hf, ours in (("self_attn_layer_norm", "ln1"), ("encoder_attn_layer_norm", "ln2"), ("final_layer_norm", "ln3")):
            st.write(d + ours + "_w", st.take(p + hf + ".weight"))
            st.write(d + ours + "_b", st.take(p + hf + ".bias"))
        for n in ("fc1", "fc2"):
            st.write(d + n + "_w", st.take(p + n + ".weight"))
            st.write(d + n + "_b", st.take(p + n + ".bias"))
    st.write("lnf_w", st.take("layer_norm.weight"))
    st.write("lnf_b", st.take("layer_norm.bias"))
    head = full.get("proj_out.weight")
    if head is not None and "embed_tokens.weight" in T and not torch.equal(head, T["embed_tokens.weight"]):
        st.bad.append("proj_out.weight differs from the token embedding (untied heads are not supported)")
    return st.done()


@torch.no_grad()
def load_higgs_audio_tower(enc, proj, src) -> dict:
    """The audio tower (``audio_tower.*``: Whisper encoder names, position table included) and the projector
    (``audio_encoder_proj.temporal`` depthwise convolution, ``linear1`` / ``linear2``) of a Higgs-Audio speech-to-text
    checkpoint. Reference: mstar/model/higgs_audio/components/audio_tower.py:27-87."""
    T = _tensors_of(src)
    res = load_whisper_encoder(enc, {k: v for k, v in T.items() if k.startswith("audio_tower.")}, prefix="audio_tower.")
    pre = "audio_encoder_proj."
    st = _Strict(proj, {k[len(pre):]: v for k, v in T.items() if k.startswith(pre)}, "Higgs-Audio projector")
    for a, b in (("temporal.weight", "temporal.weight"), ("temporal.bias", "temporal.bias"), ("linear1.weight", "w1"),
                 ("linear1.bias", "b1"), ("linear2.weight", "w2"), ("linear2.bias", "b2")):
        st.write(b, st.take(a))
    res2 = st.done()
    return {"tower": res, "projector": res2}


# ------------------------------------------------------------------ SigLIP vision tower (Hugging Face names)
@torch.no_grad()
def load_siglip_vision(enc, src, prefix: str = "vision_model.", position_table: bool = True) -> dict:
    """``VisionEncoder`` (learned positions, pre-LN blocks, tanh-GELU MLP) from a Hugging Face ``SiglipVisionModel``
    checkpoint — the vision tower of BAGEL and of the PaliGemma-based policies. The Conv2d patch embedding becomes a
    GEMM weight over flattened patches; the position table must have the encoder's ``pos_grid``² rows. The pooling
    head of the checkpoint (``head.*``), when present, is not used by these models and is ignored; a projector
    (``proj1`` / ``proj2``) of the encoder is not part of this layout: the caller loads it. ``position_table=False``
    leaves the position table to the caller as well (BAGEL keeps its own NaViT table next to the tower)."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(enc, T, "SigLIP vision tower")
    w = st.take("embeddings.patch_embedding.weight")
    st.write("patch_w", None if w is None else w.reshape(w.shape[0], -1))
    st.write("patch_b", st.take("embeddings.patch_embedding.bias"))
    if position_table:
        st.write("pos_table", st.take("embeddings.position_embedding.weight"))
    else:
        st.take("embeddings.position_embedding.weight", optional=True)
    for i in range(len(enc.enc.layers)):
        p, d = f"encoder.layers.{i}.", f"enc.layers.{i}."
        ws = [st.take(f"{p}self_attn.{n}_proj.weight") for n in "qkv"]
        bs = [st.take(f"{p}self_attn.{n}_proj.bias") for n in "qkv"]
        if None not in ws and None not in bs:
            st.write(d + "qkv_w", torch.cat(ws))
            st.write(d + "qkv_b", torch.cat(bs))
        st.write(d + "o_w", st.take(p + "self_attn.out_proj.weight"))
        st.write(d + "o_b", st.take(p + "self_attn.out_proj.bias"))
        for hf, ours in (("layer_norm1", "n1"), ("layer_norm2", "n2")):
            st.write(d + ours + "_w", st.take(p + hf + ".weight"))
            st.write(d + ours + "_b", st.take(p + hf + ".bias"))
        for n in ("fc1", "fc2"):
            st.write(d + n + "_w", st.take(f"{p}mlp.{n}.weight"))
            st.write(d + n + "_b", st.take(f"{p}mlp.{n}.bias"))
    st.write("enc.fn_w", st.take("post_layernorm.weight"))
    st.write("enc.fn_b", st.take("post_layernorm.bias"))
    return st.done(ignore_keys=("head.",), ignore_params=("proj",) + (() if position_table else ("pos_table",)))


# ------------------------------------------------------------------ BAGEL mixture-of-transformers (original names)
_BAGEL_SIDE = {"vae2llm.weight": "vae2llm_w", "vae2llm.bias": "vae2llm_b", "llm2vae.weight": "llm2vae_w",
               "llm2vae.bias": "llm2vae_b", "time_embedder.mlp.0.weight": "t1_w", "time_embedder.mlp.0.bias": "t1_b",
               "time_embedder.mlp.2.weight": "t2_w", "time_embedder.mlp.2.bias": "t2_b"}
# fixed sine-cosine tables stored as frozen parameters (computed on the fly here) and the parts that other nodes load
_BAGEL_IGNORE = ("latent_pos_embed.", "vit_pos_embed.", "vit_model.", "connector.")


@torch.no_grad()
def load_bagel_mot(m, src) -> dict:
    """``BagelMoT`` (understanding expert ``und`` + generation expert ``gen`` + latent / timestep projections) from the
    published BAGEL ``ema.safetensors`` names: ``language_model.model.layers.N.*`` with the generation expert's
    copies under ``*_moe_gen``, unfused q / k / v (+ biases) and gate / up, per-head ``q_norm`` / ``k_norm``. One
    tensor-parallel rank (the reference does not shard BAGEL either). Strict."""
    from ..ops import gemm
    import re
    T = _tensors_of(src)
    st = _Strict(m, T, "BAGEL mixture of transformers")
    L = "language_model.model."
    st.write("und.embed_tokens", st.take(L + "embed_tokens.weight"))
    st.write("und.norm", st.take(L + "norm.weight"))
    st.write("gen.final_norm", st.take(L + "norm_moe_gen.weight"))
    if m.und.lm_head is not None:
        st.write("und.lm_head", st.take("language_model.lm_head.weight"))
    else:
        st.take("language_model.lm_head.weight", optional=True)
    for ckpt, name in _BAGEL_SIDE.items():
        st.write(name, st.take(ckpt))
    qk_norm = m.cfg.qk_norm
    for i in range(m.cfg.num_layers):
        for sfx, dst, attn, mlp in (("", f"und.layers.{i}.", "self_attn.", "mlp."), ("_moe_gen", f"gen.layers.{i}.", "", "")):
            p = f"{L}layers.{i}."
            ws = [st.take(f"{p}self_attn.{n}_proj{sfx}.weight") for n in "qkv"]
            bs = [st.take(f"{p}self_attn.{n}_proj{sfx}.bias") for n in "qkv"]
            if None not in ws and None not in bs:
                st.write(dst + attn + "qkv_proj", torch.cat(ws))
                st.write(dst + attn + "qkv_bias", torch.cat(bs))
            st.write(dst + attn + "o_proj", st.take(f"{p}self_attn.o_proj{sfx}.weight"))
            if qk_norm:
                st.write(dst + attn + "q_norm", st.take(f"{p}self_attn.q_norm{sfx}.weight"))
                st.write(dst + attn + "k_norm", st.take(f"{p}self_attn.k_norm{sfx}.weight"))
            g, u = st.take(f"{p}mlp{sfx}.gate_proj.weight"), st.take(f"{p}mlp{sfx}.up_proj.weight")
            if g is not None and u is not None:
                st.write(dst + mlp + "gate_up_proj", gemm.interleave_gate_up(g, u))
            st.write(dst + mlp + "down_proj", st.take(f"{p}mlp{sfx}.down_proj.weight"))
            und = sfx == ""
            st.write(dst + ("input_layernorm" if und else "input_norm"), st.take(f"{p}input_layernorm{sfx}.weight"))
            st.write(dst + ("post_attention_layernorm" if und else "post_norm"),
                     st.take(f"{p}post_attention_layernorm{sfx}.weight"))
    return st.done(ignore_keys=_BAGEL_IGNORE)


def bagel_checkpoint_keys(m) -> dict[str, torch.Tensor]:
    """The published key layout of a ``BagelMoT``'s weights (inverse of ``load_bagel_mot``)."""
    from ..ops import gemm
    cfg = m.cfg
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    sd = {k: v.detach().clone() for k, v in m.named_parameters()}
    L = "language_model.model."
    out = {L + "embed_tokens.weight": sd["und.embed_tokens"], L + "norm.weight": sd["und.norm"],
           L + "norm_moe_gen.weight": sd["gen.final_norm"]}
    if "und.lm_head" in sd:
        out["language_model.lm_head.weight"] = sd["und.lm_head"]
    out.update({ck_: sd[name] for ck_, name in _BAGEL_SIDE.items()})
    for i in range(cfg.num_layers):
        for sfx, dst, attn, mlp in (("", f"und.layers.{i}.", "self_attn.", "mlp."), ("_moe_gen", f"gen.layers.{i}.", "", "")):
            p = f"{L}layers.{i}."
            w, b = sd[dst + attn + "qkv_proj"], sd[dst + attn + "qkv_bias"]
            cuts = {"q": (0, Hq * D), "k": (Hq * D, (Hq + Hkv) * D), "v": ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)}
            for n, (a, e) in cuts.items():
                out[f"{p}self_attn.{n}_proj{sfx}.weight"] = w[a:e].clone()
                out[f"{p}self_attn.{n}_proj{sfx}.bias"] = b[a:e].clone()
            out[f"{p}self_attn.o_proj{sfx}.weight"] = sd[dst + attn + "o_proj"]
            if cfg.qk_norm:
                out[f"{p}self_attn.q_norm{sfx}.weight"] = sd[dst + attn + "q_norm"]
                out[f"{p}self_attn.k_norm{sfx}.weight"] = sd[dst + attn + "k_norm"]
            g, u = gemm.split_gate_up(sd[dst + mlp + "gate_up_proj"])
            out[f"{p}mlp{sfx}.gate_proj.weight"], out[f"{p}mlp{sfx}.up_proj.weight"] = g, u
            out[f"{p}mlp{sfx}.down_proj.weight"] = sd[dst + mlp + "down_proj"]
            und = sfx == ""
            out[f"{p}input_layernorm{sfx}.weight"] = sd[dst + ("input_layernorm" if und else "input_norm")]
            out[f"{p}post_attention_layernorm{sfx}.weight"] = sd[dst + ("post_attention_layernorm" if und else "post_norm")]
    return out


# ------------------------------------------------------------------ image autoencoder (latent-diffusion names)
def _ae_conv(st: _Strict, src: str, dst: str) -> None:
    st.write(dst + ".weight", st.take(src + ".weight"))
    st.write(dst + ".bias", st.take(src + ".bias"))


def _ae_res(st: _Strict, src: str, dst: str, res) -> None:
    for a, b in (("norm1", "n1"), ("norm2", "n2")):
        _ae_conv(st, f"{src}.{a}", f"{dst}.{b}")
    for a, b in (("conv1", "c1"), ("conv2", "c2")):
        _ae_conv(st, f"{src}.{a}", f"{dst}.{b}.conv")
    if res.skip is not None:
        _ae_conv(st, f"{src}.nin_shortcut", f"{dst}.skip.conv")


def _ae_mid(st: _Strict, src: str, dst: str, mid) -> None:
    _ae_res(st, src + ".block_1", dst + ".0", mid[0])
    _ae_conv(st, src + ".attn_1.norm", dst + ".1.norm")
    ws = [st.take(f"{src}.attn_1.{n}.weight") for n in "qkv"]          # 1x1 convolutions -> one stacked projection
    bs = [st.take(f"{src}.attn_1.{n}.bias") for n in "qkv"]
    if None not in ws and None not in bs:
        if len({tuple(w.shape) for w in ws}) > 1:
            st.bad.append(f"{src}.attn_1: q / k / v of different shapes {[tuple(w.shape) for w in ws]}")
        else:
            st.write(dst + ".1.qkv.weight", torch.cat([w.reshape(w.shape[0], -1) for w in ws]))
            st.write(dst + ".1.qkv.bias", torch.cat(bs))
    w = st.take(src + ".attn_1.proj_out.weight")
    st.write(dst + ".1.proj.weight", None if w is None else w.reshape(w.shape[0], -1))
    st.write(dst + ".1.proj.bias", st.take(src + ".attn_1.proj_out.bias"))
    _ae_res(st, src + ".block_2", dst + ".2", mid[2])


def _ae_names(vae):
    """(checkpoint prefix, parameter prefix, module) of every residual block and resampling conv of a 2D ``ConvVAE``
    in the latent-diffusion numbering: ``encoder.down.L.block.J`` / ``.downsample``; ``decoder.up.L.block.J`` /
    ``.upsample`` with L counted from the full-resolution end while the modules run from the coarse end."""
    from .vae import _Res, _Up
    c = vae.cfg
    n_lv = len(c.channel_mult)
    out, it = [], iter(enumerate(vae.encoder.down))
    for lv in range(n_lv):
        for j in range(c.num_res_blocks):
            i, m = next(it)
            out.append((f"encoder.down.{lv}.block.{j}", f"encoder.down.{i}", m))
        if lv < n_lv - 1:
            i, m = next(it)
            out.append((f"encoder.down.{lv}.downsample.conv", f"encoder.down.{i}.conv", m))
    it = iter(enumerate(vae.decoder.up))
    for lv in reversed(range(n_lv)):
        for j in range(c.num_res_blocks + 1):
            i, m = next(it)
            out.append((f"decoder.up.{lv}.block.{j}", f"decoder.up.{i}", m))
        if lv > 0:
            i, m = next(it)
            out.append((f"decoder.up.{lv}.upsample.conv", f"decoder.up.{i}.conv.conv", m))
    assert all(isinstance(m, _Res) or isinstance(m, _Up) or hasattr(m, "conv") for _, _, m in out)
    return out


@torch.no_grad()
def load_image_autoencoder(vae, src) -> dict:
    """2D ``ConvVAE`` from the latent-diffusion autoencoder layout that BAGEL publishes as ``ae.safetensors``
    (``encoder.down.L.block.J.{norm1,conv1,norm2,conv2,nin_shortcut}``, ``down.L.downsample.conv``,
    ``mid.{block_1,attn_1,block_2}``, ``norm_out``, ``conv_out``; the decoder mirrors it with ``up.L``). The mid-block
    attention's q / k / v / proj_out 1x1 convolutions become two linear layers. Strict.
    Reference module: mstar/model/bagel/components/autoencoder.py:107-257."""
    from .vae import _Res
    if vae.cfg.dims != 2:
        raise CheckpointMismatch("the latent-diffusion image autoencoder layout is 2D")
    st = _Strict(vae, _tensors_of(src), "image autoencoder")
    for half, mod in (("encoder", vae.encoder), ("decoder", vae.decoder)):
        _ae_conv(st, half + ".conv_in", half + ".inp.conv")
        _ae_mid(st, half + ".mid", half + ".mid", mod.mid)
        _ae_conv(st, half + ".norm_out", half + ".norm")
        _ae_conv(st, half + ".conv_out", half + ".out.conv")
    for ck, name, m in _ae_names(vae):
        if isinstance(m, _Res):
            _ae_res(st, ck, name, m)
        else:
            _ae_conv(st, ck, name)
    return st.done()


# ------------------------------------------------------------------ Pi0.5 policy (lerobot names)
_PI05_PALI = "paligemma_with_expert.paligemma.model."
_PI05_EXPERT = "paligemma_with_expert.gemma_expert.model."
_PI05_TOP = {"action_in_proj.weight": "a_in_w", "action_in_proj.bias": "a_in_b", "action_out_proj.weight": "a_out_w",
             "action_out_proj.bias": "a_out_b", "time_mlp_in.weight": "t1_w", "time_mlp_in.bias": "t1_b",
             "time_mlp_out.weight": "t2_w", "time_mlp_out.bias": "t2_b"}


def _gemma_layer(st: _Strict, src: str, dst: str, adaptive: bool) -> None:
    q, k, v = (st.take(f"{src}self_attn.{n}_proj.weight") for n in "qkv")
    if None not in (q, k, v):
        st.write(dst + "qkv", torch.cat([q, k, v]))
    st.write(dst + "o", st.take(src + "self_attn.o_proj.weight"))
    g, u = st.take(src + "mlp.gate_proj.weight"), st.take(src + "mlp.up_proj.weight")
    if g is not None and u is not None:
        st.write(dst + "gate_up", torch.cat([g, u]))                     # gate rows, then up rows
    st.write(dst + "down", st.take(src + "mlp.down_proj.weight"))
    for ck_, ours in (("input_layernorm", "1"), ("post_attention_layernorm", "2")):
        if adaptive:                # dense: condition -> (scale, shift, gate)
            st.write(f"{dst}mod{ours}_w", st.take(f"{src}{ck_}.dense.weight"))
            st.write(f"{dst}mod{ours}_b", st.take(f"{src}{ck_}.dense.bias"))
        else:
            st.write(f"{dst}n{ours}", st.take(f"{src}{ck_}.weight"))


@torch.no_grad()
def load_pi05_policy(m, src) -> dict:
    """``Pi05Policy`` (PaliGemma prefix tower ``und``, adaptive-norm action expert ``act``, action / time projections)
    from the published lerobot layout: ``paligemma_with_expert.paligemma.model.language_model.*`` and
    ``paligemma_with_expert.gemma_expert.model.*`` in Hugging Face Gemma names, the expert's norms as
    ``*.dense.{weight,bias}``, the tied token table under ``paligemma.lm_head.weight``, ``action_in_proj``,
    ``action_out_proj``, ``time_mlp_in`` / ``time_mlp_out``. The vision tower and projector are another node's
    (``load_pi05_vision``); the expert's unused ``lm_head`` / token table are ignored. Strict.
    Reference key map: mstar/model/pi05/pi05_model.py:300-347."""
    T = {k: v for k, v in _tensors_of(src).items()
         if not k.startswith((_PI05_PALI + "vision_tower.", _PI05_PALI + "multi_modal_projector."))}
    st = _Strict(m, T, "Pi0.5 policy")
    head = st.take("paligemma_with_expert.paligemma.lm_head.weight", optional=True)
    table = st.take(_PI05_PALI + "language_model.embed_tokens.weight", optional=True)
    if head is None and table is None:
        st.bad.append("missing the token table (paligemma.lm_head.weight / language_model.embed_tokens.weight)")
    st.write("embed", head if head is not None else table)
    for ck_, name in _PI05_TOP.items():
        st.write(name, st.take(ck_))
    for i in range(len(m.und.layers)):
        _gemma_layer(st, f"{_PI05_PALI}language_model.layers.{i}.", f"und.layers.{i}.", False)
        _gemma_layer(st, f"{_PI05_EXPERT}layers.{i}.", f"act.layers.{i}.", True)
    st.write("und.nf", st.take(_PI05_PALI + "language_model.norm.weight"))
    st.write("act.modf_w", st.take(_PI05_EXPERT + "norm.dense.weight"))
    st.write("act.modf_b", st.take(_PI05_EXPERT + "norm.dense.bias"))
    return st.done(ignore_keys=("paligemma_with_expert.gemma_expert.lm_head.weight", _PI05_EXPERT + "embed_tokens.weight"))


@torch.no_grad()
def load_pi05_vision(enc, src) -> dict:
    """The policy's camera encoder from the same file: SigLIP names under
    ``paligemma_with_expert.paligemma.model.vision_tower.vision_model.`` and the one-layer projector under
    ``…multi_modal_projector.linear``. Strict over those two prefixes.
    Reference: mstar/model/pi05/pi05_model.py:349-377."""
    T = _tensors_of(src)
    vt, mp = _PI05_PALI + "vision_tower.vision_model.", _PI05_PALI + "multi_modal_projector.linear."
    w, b = T.get(mp + "weight"), T.get(mp + "bias")
    for t, p, n in ((w, enc.proj2_w, "weight"), (b, enc.proj2_b, "bias")):
        if t is None or tuple(t.shape) != tuple(p.shape):
            raise CheckpointMismatch(f"Pi0.5 vision projector: {mp}{n} missing or of shape "
                                     f"{None if t is None else tuple(t.shape)} (parameter {tuple(p.shape)})")
        p.data.copy_(t.to(p.dtype))
    return load_siglip_vision(enc, {k[len(vt):]: v for k, v in T.items() if k.startswith(vt)}, prefix="")


def pi05_checkpoint_keys(m, enc=None) -> dict[str, torch.Tensor]:
    """The published key layout of a ``Pi05Policy`` (and, with ``enc``, of its camera encoder's projector): inverse
    of ``load_pi05_policy``."""
    sd = {k: v.detach().clone() for k, v in m.named_parameters()}
    nh, nkv, D = m.und.nh, m.und.nkv, m.und.D
    out = {"paligemma_with_expert.paligemma.lm_head.weight": sd["embed"]}
    out.update({ck_: sd[name] for ck_, name in _PI05_TOP.items()})
    for tower, pre, adaptive in (("und", _PI05_PALI + "language_model.", False), ("act", _PI05_EXPERT, True)):
        for i in range(len(m.und.layers)):
            s, d = f"{tower}.layers.{i}.", f"{pre}layers.{i}."
            qkv = sd[s + "qkv"]
            out[d + "self_attn.q_proj.weight"] = qkv[:nh * D].clone()
            out[d + "self_attn.k_proj.weight"] = qkv[nh * D:(nh + nkv) * D].clone()
            out[d + "self_attn.v_proj.weight"] = qkv[(nh + nkv) * D:].clone()
            out[d + "self_attn.o_proj.weight"] = sd[s + "o"]
            gu = sd[s + "gate_up"]
            out[d + "mlp.gate_proj.weight"], out[d + "mlp.up_proj.weight"] = gu[:gu.shape[0] // 2].clone(), gu[gu.shape[0] // 2:].clone()
            out[d + "mlp.down_proj.weight"] = sd[s + "down"]
            for ck_, ours in (("input_layernorm", "1"), ("post_attention_layernorm", "2")):
                if adaptive:
                    out[f"{d}{ck_}.dense.weight"], out[f"{d}{ck_}.dense.bias"] = sd[f"{s}mod{ours}_w"], sd[f"{s}mod{ours}_b"]
                else:
                    out[f"{d}{ck_}.weight"] = sd[f"{s}n{ours}"]
    out[_PI05_PALI + "language_model.norm.weight"] = sd["und.nf"]
    out[_PI05_EXPERT + "norm.dense.weight"], out[_PI05_EXPERT + "norm.dense.bias"] = sd["act.modf_w"], sd["act.modf_b"]
    return out


# ------------------------------------------------------------------ Qwen3-Omni towers (Hugging Face names)
@torch.no_grad()
def load_qwen3_omni_audio(enc, src, prefix: str = "thinker.audio_tower.") -> dict:
    """``OmniAudioEncoder`` from the ``thinker.audio_tower.*`` tensors of a Qwen3-Omni checkpoint: three Conv2d,
    ``conv_out``, Whisper-named layers (separate q / k / v with biases), ``ln_post``, ``proj1`` / ``proj2``. Strict
    over the prefix. Reference: mstar/model/qwen3_omni/qwen3_omni_model.py:1507-1539."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(enc, T, "Qwen3-Omni audio tower")
    for n in ("conv2d1", "conv2d2", "conv2d3"):
        st.write(n + ".weight", st.take(n + ".weight"))
        st.write(n + ".bias", st.take(n + ".bias"))
    st.write("conv_out_w", st.take("conv_out.weight"))
    for i in range(len(enc.enc.layers)):
        p, d = f"layers.{i}.", f"enc.layers.{i}."
        ws = [st.take(f"{p}self_attn.{n}_proj.weight") for n in "qkv"]
        bs = [st.take(f"{p}self_attn.{n}_proj.bias") for n in "qkv"]
        if None not in ws and None not in bs:
            st.write(d + "qkv_w", torch.cat(ws))
            st.write(d + "qkv_b", torch.cat(bs))
        st.write(d + "o_w", st.take(p + "self_attn.out_proj.weight"))
        st.write(d + "o_b", st.take(p + "self_attn.out_proj.bias"))
        for hf, ours in (("self_attn_layer_norm", "n1"), ("final_layer_norm", "n2")):
            st.write(d + ours + "_w", st.take(p + hf + ".weight"))
            st.write(d + ours + "_b", st.take(p + hf + ".bias"))
        for n in ("fc1", "fc2"):
            st.write(d + n + "_w", st.take(f"{p}{n}.weight"))
            st.write(d + n + "_b", st.take(f"{p}{n}.bias"))
    st.write("enc.fn_w", st.take("ln_post.weight"))
    st.write("enc.fn_b", st.take("ln_post.bias"))
    for n in ("proj1", "proj2"):
        st.write(n + "_w", st.take(n + ".weight"))
        st.write(n + "_b", st.take(n + ".bias"))
    return st.done()


def _omni_merger(st: _Strict, src: str, dst: str) -> None:
    st.write(dst + "norm_w", st.take(src + "ln_q.weight"))
    st.write(dst + "norm_b", st.take(src + "ln_q.bias"))
    for hf, ours in (("mlp.0", "fc1"), ("mlp.2", "fc2")):
        st.write(f"{dst}{ours}_w", st.take(f"{src}{hf}.weight"))
        st.write(f"{dst}{ours}_b", st.take(f"{src}{hf}.bias"))


@torch.no_grad()
def load_qwen3_omni_vision(enc, src, prefix: str = "thinker.visual.") -> dict:
    """``OmniVisionEncoder`` from the ``thinker.visual.*`` tensors of a Qwen3-Omni checkpoint: Conv3d patch embedding
    (flattened to a GEMM weight), the learned position table, blocks with a fused ``attn.qkv``, ``merger`` and the
    deepstack ``merger_list``. Strict over the prefix. Reference: mstar/model/qwen3_omni/qwen3_omni_model.py:1546-1580."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(enc, T, "Qwen3-Omni vision tower")
    w = st.take("patch_embed.proj.weight")
    st.write("patch_w", None if w is None else w.reshape(w.shape[0], -1))
    st.write("patch_b", st.take("patch_embed.proj.bias"))
    st.write("pos_table", st.take("pos_embed.weight"))
    for i in range(len(enc.enc.layers)):
        p, d = f"blocks.{i}.", f"enc.layers.{i}."
        for hf, ours in (("norm1", "n1"), ("norm2", "n2"), ("attn.qkv", "qkv"), ("attn.proj", "o"),
                         ("mlp.linear_fc1", "fc1"), ("mlp.linear_fc2", "fc2")):
            st.write(f"{d}{ours}_w", st.take(f"{p}{hf}.weight"))
            st.write(f"{d}{ours}_b", st.take(f"{p}{hf}.bias"))
    _omni_merger(st, "merger.", "merger.")
    for k in range(len(enc.deep_mergers)):
        _omni_merger(st, f"merger_list.{k}.", f"deep_mergers.{k}.")
    return st.done()


@torch.no_grad()
def load_qwen3_omni_code2wav(m, src, prefix: str = "code2wav.") -> dict:
    """``OmniCode2Wav`` from the ``code2wav.*`` tensors of a Qwen3-Omni checkpoint: ``code_embedding``,
    ``pre_transformer`` (Hugging Face decoder names plus the two ``*_layer_scale.scale`` vectors),
    ``upsample.N.{0,1}`` and the ``decoder.N`` list (input convolution, up blocks ``block.0 … block.4``, final
    activation and convolution). Strict over the prefix.
    Reference module: mstar/model/qwen3_omni/components/code2wav.py."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(m, T, "Qwen3-Omni code2wav")

    def same(src_, dst, names):
        for n in names:
            st.write(f"{dst}.{n}", st.take(f"{src_}.{n}"))
    wb, ab = ("weight", "bias"), ("alpha", "beta")
    st.write("code_embedding", st.take("code_embedding.weight"))
    for i in range(len(m.pre.layers)):
        p, d = f"pre_transformer.layers.{i}.", f"pre.layers.{i}."
        ws = [st.take(f"{p}self_attn.{n}_proj.weight") for n in "qkv"]
        if None not in ws:
            st.write(d + "qkv", torch.cat(ws))
        st.write(d + "o", st.take(p + "self_attn.o_proj.weight"))
        g, u = st.take(p + "mlp.gate_proj.weight"), st.take(p + "mlp.up_proj.weight")
        if g is not None and u is not None:
            st.write(d + "gate_up", torch.cat([g, u]))
        st.write(d + "down", st.take(p + "mlp.down_proj.weight"))
        st.write(d + "n1", st.take(p + "input_layernorm.weight"))
        st.write(d + "n2", st.take(p + "post_attention_layernorm.weight"))
        st.write(d + "s1", st.take(p + "self_attn_layer_scale.scale"))
        st.write(d + "s2", st.take(p + "mlp_layer_scale.scale"))
    st.write("pre.norm", st.take("pre_transformer.norm.weight"))
    for i in range(len(m.upsample)):
        same(f"upsample.{i}.0.conv", f"upsample.{i}.0.conv", wb)
        same(f"upsample.{i}.1.dwconv.conv", f"upsample.{i}.1.dwconv.conv", wb)
        for n in ("norm", "pwconv1", "pwconv2"):
            same(f"upsample.{i}.1.{n}", f"upsample.{i}.1.{n}", wb)
        st.write(f"upsample.{i}.1.gamma", st.take(f"upsample.{i}.1.gamma"))
    same("decoder.0.conv", "inp.conv", wb)
    nb = len(m.blocks)
    for i in range(nb):
        p, d = f"decoder.{i + 1}.block.", f"blocks.{i}."
        same(p + "0", d + "act", ab)
        same(p + "1.conv", d + "up.conv", wb)
        for r in range(3):
            q, e = f"{p}{r + 2}.", f"{d}res.{r}."
            same(q + "act1", e + "act1", ab)
            same(q + "conv1.conv", e + "conv1.conv", wb)
            same(q + "act2", e + "act2", ab)
            same(q + "conv2.conv", e + "conv2.conv", wb)
    same(f"decoder.{nb + 1}", "out_act", ab)
    same(f"decoder.{nb + 2}.conv", "out.conv", wb)
    return st.done()


# ------------------------------------------------------------------ V-JEPA 2 (Hugging Face names)
def _vjepa2_layers(st: _Strict, n: int, src: str, dst: str) -> None:
    for i in range(n):
        p, d = f"{src}layer.{i}.", f"{dst}layers.{i}."
        ws = [st.take(f"{p}attention.{n_}.weight") for n_ in ("query", "key", "value")]
        bs = [st.take(f"{p}attention.{n_}.bias") for n_ in ("query", "key", "value")]
        if None not in ws and None not in bs:
            st.write(d + "qkv_w", torch.cat(ws))
            st.write(d + "qkv_b", torch.cat(bs))
        for hf, ours in (("attention.proj", "o"), ("norm1", "n1"), ("norm2", "n2"), ("mlp.fc1", "fc1"), ("mlp.fc2", "fc2")):
            st.write(f"{d}{ours}_w", st.take(f"{p}{hf}.weight"))
            st.write(f"{d}{ours}_b", st.take(f"{p}{hf}.bias"))
    st.write(dst + "fn_w", st.take(src + "layernorm.weight"))
    st.write(dst + "fn_b", st.take(src + "layernorm.bias"))


@torch.no_grad()
def load_vjepa2_encoder(enc, src, prefix: str = "encoder.") -> dict:
    """``VJepa2Encoder`` from the ``encoder.*`` tensors of a Hugging Face V-JEPA 2 checkpoint
    (``facebook/vjepa2-vit*-fpc64-*``): Conv3d tubelet embedding flattened to a GEMM weight, separate query / key /
    value projections stacked. Strict over the prefix. Reference: mstar/model/vjepa2/weight_loader.py:1-60."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(enc, T, "V-JEPA 2 encoder")
    w = st.take("embeddings.patch_embeddings.proj.weight")
    st.write("patch_w", None if w is None else w.reshape(w.shape[0], -1))
    st.write("patch_b", st.take("embeddings.patch_embeddings.proj.bias"))
    _vjepa2_layers(st, len(enc.enc.layers), "", "enc.")
    return st.done()


@torch.no_grad()
def load_vjepa2_predictor(pred, src, prefix: str = "predictor.") -> dict:
    """``MaskedPredictor`` from the ``predictor.*`` tensors of the same checkpoint: ``predictor_embeddings``, the mask
    tokens ([n, 1, 1, hidden] -> [n, hidden]), the layers, ``layernorm`` and ``proj``. Strict over the prefix."""
    T = {k[len(prefix):]: v for k, v in _tensors_of(src).items() if k.startswith(prefix)}
    st = _Strict(pred, T, "V-JEPA 2 predictor")
    st.write("inp_w", st.take("embeddings.predictor_embeddings.weight"))
    st.write("inp_b", st.take("embeddings.predictor_embeddings.bias"))
    m = st.take("embeddings.mask_tokens")
    st.write("mask_tokens", None if m is None else m.reshape(m.shape[0], -1))
    _vjepa2_layers(st, len(pred.blocks.layers), "", "blocks.")
    st.write("out_w", st.take("proj.weight"))
    st.write("out_b", st.take("proj.bias"))
    return st.done()


# ------------------------------------------------------------------ SNAC decoder (published names)
def _fold_weight_norm(T: dict, key: str) -> torch.Tensor | None:
    """The plain weight of a weight-normalised convolution: ``key.weight`` if stored, else g * v / ||v|| from
    ``key.parametrizations.weight.original{0,1}`` or the older ``key.weight_{g,v}`` (norm over all but dim 0)."""
    if key + ".weight" in T:
        return T.pop(key + ".weight")
    for g_name, v_name in ((".parametrizations.weight.original0", ".parametrizations.weight.original1"),
                           (".weight_g", ".weight_v")):
        if key + g_name in T and key + v_name in T:
            g, v = T.pop(key + g_name).float(), T.pop(key + v_name).float()
            return g * v / v.flatten(1).norm(dim=1).reshape(-1, *([1] * (v.dim() - 1)))
    return None


@torch.no_grad()
def load_snac_decoder(dec, src) -> dict:
    """``SnacDecoder`` from the published SNAC checkpoint (``pytorch_model.bin`` of ``hubertsiuzdak/snac_24khz``, a
    directory holding it, or its state dict): codebooks and their output projections, the decoder's
    ``decoder.model.N`` list (input convolutions, up blocks with noise projection and three residual units, final
    activation and convolution). Weight normalisation is folded into plain weights; the encoder and the quantiser's
    input projections are not part of a decoder and are ignored. Strict over everything else.
    Reference: mstar/model/orpheus/components/snac.py:239-272, 317-358, 399-424."""
    import os
    if isinstance(src, str):
        path = os.path.join(src, "pytorch_model.bin") if os.path.isdir(src) else src
        raw = torch.load(path, map_location="cpu", weights_only=True)
    else:
        raw = dict(src)
    T = {k: v for k, v in raw.items() if not k.startswith("encoder.") and ".in_proj." not in k}
    params = dict(dec.named_parameters())
    written: set[str] = set()
    bad: list[str] = []

    def put(name: str, t: torch.Tensor | None, what: str) -> None:
        p = params.get(name)
        if t is None or p is None or tuple(p.shape) != tuple(t.shape):
            bad.append(f"{what} -> {name}: {None if t is None else tuple(t.shape)} vs {None if p is None else tuple(p.shape)}")
            return
        p.copy_(t.to(p.dtype))
        written.add(name)

    def conv(src_, dst, bias=True):
        put(dst + ".weight", _fold_weight_norm(T, src_), src_)
        if bias:
            put(dst + ".bias", T.pop(src_ + ".bias", None), src_ + ".bias")

    for i in range(len(dec.codebooks)):
        q = f"quantizer.quantizers.{i}."
        put(f"codebooks.{i}.weight", T.pop(q + "codebook.weight", None), q + "codebook.weight")
        conv(q + "out_proj", f"out_proj.{i}")
    n = 0
    if isinstance(dec.inp, torch.nn.Sequential):
        conv("decoder.model.0", "inp.0")
        conv("decoder.model.1", "inp.1")
        n = 2
    else:
        conv("decoder.model.0", "inp")
        n = 1
    for i, blk in enumerate(dec.blocks):
        b = f"decoder.model.{n + i}.block."
        put(f"blocks.{i}.up.0.alpha", T.pop(b + "0.alpha", None), b + "0.alpha")
        conv(b + "1", f"blocks.{i}.up.1")
        k = 2
        if blk.noise is not None:
            conv(b + "2.linear", f"blocks.{i}.noise", bias=False)
            k = 3
        for r in range(3):
            u, d = f"{b}{k + r}.block.", f"blocks.{i}.res.{r}.block."
            put(d + "0.alpha", T.pop(u + "0.alpha", None), u + "0.alpha")
            conv(u + "1", d + "1")
            put(d + "2.alpha", T.pop(u + "2.alpha", None), u + "2.alpha")
            conv(u + "3", d + "3")
    n += len(dec.blocks)
    put("out.0.alpha", T.pop(f"decoder.model.{n}.alpha", None), f"decoder.model.{n}.alpha")
    conv(f"decoder.model.{n + 1}", "out.1")
    missing = sorted(set(params) - written)
    if T or missing or bad:
        raise CheckpointMismatch(f"SNAC decoder: {len(T)} checkpoint tensors without a parameter {sorted(T)[:5]}, "
                                 f"{len(missing)} parameters not loaded {missing[:5]}, problems {bad[:5]}")
    return {"loaded": len(written)}


@torch.no_grad()
def load_qwen3_omni_code_predictor(pred, src, prefix: str = "talker.code_predictor.",
                                   talker_table: str = "talker.model.codec_embedding.weight") -> dict:
    """``CodePredictor`` from the ``talker.code_predictor.*`` tensors of a Qwen3-Omni checkpoint: a dense Qwen3-style
    stack (``model.layers``, ``model.norm``), one embedding table per residual code layer
    (``model.codec_embedding.N``) and one head per layer (``lm_head.N``). The first code of a frame is embedded with
    the TALKER's table (``talker_table``, its first ``codebook`` rows); the talker's hidden state enters unprojected,
    so predictor and talker must have the same width. Strict over the prefix."""
    from ..ops import gemm
    allT = _tensors_of(src)
    T = {k[len(prefix):]: v for k, v in allT.items() if k.startswith(prefix)}
    st = _Strict(pred, T, "Qwen3-Omni code predictor")
    H = pred.cfg.hidden_size
    if tuple(pred.in_proj.shape) != (H, H):
        st.bad.append(f"the talker's width {pred.in_proj.shape[1]} differs from the predictor's {H}")
    else:
        st.write("in_proj", torch.eye(H))
    tbl = allT.get(talker_table)
    embeds = [None if tbl is None else tbl[:pred.codebook]]
    embeds += [st.take(f"model.codec_embedding.{j}.weight") for j in range(pred.n_sub)]
    if any(e is None for e in embeds):
        st.bad.append(f"missing {talker_table} or a codec_embedding table")
    else:
        st.write("embed", torch.stack([e[:pred.codebook] for e in embeds]))
    heads = [st.take(f"lm_head.{j}.weight") for j in range(pred.n_sub)]
    if None not in heads:
        st.write("heads", torch.stack([h[:pred.codebook] for h in heads]))
    for i in range(len(pred.tower.layers)):
        p, d = f"model.layers.{i}.", f"tower.layers.{i}."
        ws = [st.take(f"{p}self_attn.{n}_proj.weight") for n in "qkv"]
        if None not in ws:
            st.write(d + "qkv_proj", torch.cat(ws))
        st.write(d + "o_proj", st.take(p + "self_attn.o_proj.weight"))
        st.write(d + "q_norm", st.take(p + "self_attn.q_norm.weight"))
        st.write(d + "k_norm", st.take(p + "self_attn.k_norm.weight"))
        g, u = st.take(p + "mlp.gate_proj.weight"), st.take(p + "mlp.up_proj.weight")
        if g is not None and u is not None:
            st.write(d + "gate_up_proj", gemm.interleave_gate_up(g, u))
        st.write(d + "down_proj", st.take(p + "mlp.down_proj.weight"))
        st.write(d + "input_norm", st.take(p + "input_layernorm.weight"))
        st.write(d + "post_norm", st.take(p + "post_attention_layernorm.weight"))
    st.write("tower.final_norm", st.take("model.norm.weight"))
    return st.done()
