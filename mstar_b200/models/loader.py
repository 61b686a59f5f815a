"""Checkpoint loading: stream tensors out of (sharded) safetensors files straight into the fused, sharded
parameters of this library's modules — q/k/v rows of the rank's heads into ``qkv_proj``, gate/up rows interleaved
into ``gate_up_proj`` (the layout the SwiGLU GEMM epilogue expects), per-expert MoE weights stacked into ``w13`` /
``w2``, row-parallel weights cut by columns. Nothing is materialised twice: one tensor is read, cut, cast and
copied at a time.

Reference counterparts: streaming iterators (mstar/model/loader/iterators.py:24-80), stacked-parameter rules and
``load_hf_weights`` (mstar/model/loader/base.py:97-230), per-model loaders such as the Qwen3-Omni per-expert fuse
(mstar/model/qwen3_omni/qwen3_omni_model.py:1297-1347).
"""
from __future__ import annotations

import json
import os
import re
from collections.abc import Callable, Iterator

import torch

from ..ops import gemm
from .decoder import DecoderLM, GatedMLP, shard_qkv


def iter_safetensors(model_dir: str, prefix: str | None = None) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, CPU tensor) for every tensor of a checkpoint directory (index file, or every *.safetensors)."""
    from safetensors import safe_open
    files: list[str]
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {model_dir}")
    for fn in files:
        with safe_open(os.path.join(model_dir, fn), framework="pt", device="cpu") as f:
            for k in f.keys():
                if prefix is None or k.startswith(prefix):
                    yield k, f.get_tensor(k)


@torch.no_grad()
def load_named_tensors(module: torch.nn.Module, model_dir: str, rename: Callable[[str], str | None] | None = None,
                       strict: bool = False) -> dict:
    """Copy checkpoint tensors into same-named parameters / buffers (after ``rename``; None drops a tensor).
    Returns {"missing": [...], "unexpected": [...]}."""
    targets = dict(module.named_parameters())
    targets.update(dict(module.named_buffers()))
    seen, unexpected = set(), []
    for name, t in iter_safetensors(model_dir):
        dst_name = rename(name) if rename else name
        if dst_name is None:
            continue
        dst = targets.get(dst_name)
        if dst is None or tuple(dst.shape) != tuple(t.shape):
            unexpected.append(name)
            continue
        dst.copy_(t.to(dst.dtype))
        seen.add(dst_name)
    missing = sorted(set(targets) - seen)
    if strict and (missing or unexpected):
        raise RuntimeError(f"checkpoint mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    return {"missing": missing, "unexpected": unexpected}


class _Pending:
    """Collects the pieces of a fused parameter until all have arrived."""

    def __init__(self):
        self.parts: dict[tuple, dict[str, torch.Tensor]] = {}

    def add(self, key: tuple, part: str, t: torch.Tensor, need: tuple[str, ...]):
        d = self.parts.setdefault(key, {})
        d[part] = t
        if all(n in d for n in need):
            return self.parts.pop(key)
        return None


@torch.no_grad()
def load_decoder_from_hf(lm: DecoderLM, model_dir: str, prefix: str = "model.", head_name: str = "lm_head.weight",
                         layer_filter: Callable[[str], str | None] | None = None, embed_name: str = "embed_tokens.weight",
                         strict: bool = True, ignore: tuple[str, ...] = ("rotary_emb.inv_freq",)) -> dict:
    """Fill a (possibly tensor-parallel) ``DecoderLM`` from a Hugging Face Llama / Qwen2 / Qwen3 / Qwen3-MoE style
    checkpoint. ``layer_filter`` may rewrite or drop names first (towers that live under another prefix, e.g.
    ``thinker.model.``); ``embed_name`` is the token table's name under the prefix (``codec_embedding.weight`` for a
    speech-token decoder). ``strict``: every parameter of the decoder must have been written (a tied head may take the
    token table) and every tensor under the prefix must have found a parameter, else ``CheckpointMismatch``; the
    result lists both in any case."""
    cfg, tp = lm.cfg, lm.tp
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    pend = _Pending()
    loaded = 0
    unused: list[str] = []
    for p_ in lm.parameters():          # a parameter that no tensor reaches still holds this after the load
        if p_.is_floating_point():
            p_.data.fill_(float("nan"))
    rx = re.compile(r"layers\.(\d+)\.(.+)")
    for name, t in iter_safetensors(model_dir):
        if layer_filter is not None:
            name = layer_filter(name)
            if name is None:
                continue
        if name == head_name:
            if lm.lm_head is not None:
                lm.lm_head.copy_(lm.vocab_rows(t.to(cfg.dtype)))
                loaded += 1
            continue
        if not name.startswith(prefix):
            continue
        key = name[len(prefix):]
        if key == embed_name:
            if lm.embed_tokens is not None:
                lm.embed_tokens.copy_(lm.vocab_rows(t.to(cfg.dtype)))
                loaded += 1
            continue
        if key == "norm.weight":
            lm.norm.copy_(t.to(cfg.dtype))
            loaded += 1
            continue
        m = rx.match(key)
        if not m or int(m.group(1)) >= len(lm.layers):
            if not key.endswith(ignore):
                unused.append(name)
            continue
        li, sub = int(m.group(1)), m.group(2)
        layer = lm.layers[li]
        at = layer.self_attn
        if sub in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            getattr(layer, sub.split(".")[0]).copy_(t.to(cfg.dtype))
        elif sub in ("self_attn.q_norm.weight", "self_attn.k_norm.weight") and at.q_norm is not None:
            getattr(at, sub.split(".")[1]).copy_(t.to(cfg.dtype))
        elif re.fullmatch(r"self_attn\.[qkv]_proj\.(weight|bias)", sub):
            which, kind = sub.split(".")[1][0], sub.split(".")[2]
            got = pend.add((li, "qkv", kind), which, t, ("q", "k", "v"))
            if got:
                fused = shard_qkv(got["q"], got["k"], got["v"], Hq, Hkv, D, tp.rank, tp.size).to(cfg.dtype)
                (at.qkv_proj if kind == "weight" else at.qkv_bias).copy_(fused)
        elif sub == "self_attn.o_proj.weight":
            at.o_proj.copy_(t[:, tp.rank * at.Hq * D:(tp.rank + 1) * at.Hq * D].to(cfg.dtype))
        elif re.fullmatch(r"mlp\.(gate|up|down)_proj\.weight", sub) and isinstance(layer.mlp, GatedMLP):
            got = pend.add((li, "mlp"), sub.split(".")[1][:-5], t, ("gate", "up", "down"))
            if got:
                F = got["gate"].shape[0] // tp.size
                sl = slice(tp.rank * F, (tp.rank + 1) * F)
                layer.mlp.gate_up_proj.copy_(gemm.interleave_gate_up(got["gate"][sl], got["up"][sl]).to(cfg.dtype))
                layer.mlp.down_proj.copy_(got["down"][:, sl].to(cfg.dtype))
        elif sub == "mlp.gate.weight" and hasattr(layer.mlp, "router"):
            layer.mlp.router.copy_(t.to(cfg.dtype))
        elif (me := re.fullmatch(r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight", sub)) and hasattr(layer.mlp, "w13"):
            e = int(me.group(1))
            lo, hi = layer.mlp.expert_range
            if not (lo <= e < hi):
                continue
            got = pend.add((li, "exp", e), me.group(2), t, ("gate", "up", "down"))
            if got:
                I = layer.mlp.I_local
                full = got["gate"].shape[0]
                r = 0 if I == full else tp.rank
                sl = slice(r * I, (r + 1) * I)
                layer.mlp.w13[e - lo].copy_(gemm.interleave_gate_up(got["gate"][sl], got["up"][sl]).to(cfg.dtype))
                layer.mlp.w2[e - lo].copy_(got["down"][:, sl].to(cfg.dtype))
        elif re.fullmatch(r"mlp\.shared_expert\.(gate|up|down)_proj\.weight", sub) and getattr(layer.mlp, "shared", None) is not None:
            got = pend.add((li, "shared"), sub.split(".")[2][:-5], t, ("gate", "up", "down"))
            if got:
                sh = layer.mlp.shared
                F = got["gate"].shape[0] // tp.size
                sl = slice(tp.rank * F, (tp.rank + 1) * F)
                sh.gate_up_proj.copy_(gemm.interleave_gate_up(got["gate"][sl], got["up"][sl]).to(cfg.dtype))
                sh.down_proj.copy_(got["down"][:, sl].to(cfg.dtype))
        elif sub == "mlp.shared_expert_gate.weight" and getattr(layer.mlp, "shared", None) is not None:
            layer.mlp.shared_gate.copy_(t.to(cfg.dtype))
        else:
            if not sub.endswith(ignore):
                unused.append(name)
            continue
        loaded += 1
    if getattr(lm, "vocab_parallel", False):
        torch.cuda.synchronize(lm.device_)
        lm.tp.symm.barrier()            # every rank's table shard is in place before anyone gathers rows from it
        torch.cuda.synchronize(lm.device_)
    # a head that the checkpoint does not store is tied to the token table
    if lm.lm_head is not None and lm.embed_tokens is not None and bool(torch.isnan(lm.lm_head).all()) \
            and lm.lm_head.shape == lm.embed_tokens.shape and not bool(torch.isnan(lm.embed_tokens).any()):
        lm.lm_head.copy_(lm.embed_tokens)
    missing = [n for n, p_ in lm.named_parameters() if p_.is_floating_point() and bool(torch.isnan(p_).any())]
    incomplete = [str(k) for k in pend.parts]
    if strict and (missing or unused or incomplete):
        from .checkpoints import CheckpointMismatch
        raise CheckpointMismatch(f"decoder checkpoint under {prefix!r}: {len(missing)} parameters not loaded {missing[:5]}, "
                                 f"{len(unused)} tensors without a parameter {unused[:5]}, incomplete fused groups "
                                 f"{incomplete[:5]}")
    return {"loaded": loaded, "incomplete": incomplete, "missing": missing, "unused": unused}
