"""The tiny Qwen-style decoder used as the standing fixture and correctness oracle: 2 layers, hidden 256,
4 query / 2 KV heads of dim 64, SwiGLU FFN 688, RMSNorm, RoPE theta 1e6, vocabulary 32000, weights N(0, 0.02)
from seed 0.

``oracle_generate`` is an independent, cache-free fp32 implementation in plain PyTorch (full recompute of the
prefix at every step) that the engine's paged, batched, kernel-backed path has to reproduce token for token.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .decoder import DecoderConfig, DecoderLM


def tiny_config(dtype=torch.float32) -> DecoderConfig:
    return DecoderConfig(hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                         intermediate_size=688, vocab_size=32000, rms_eps=1e-6, rope_theta=1e6, dtype=dtype)


def build_tiny(device="cpu", dtype=torch.float32, seed: int = 0, tp=None) -> DecoderLM:
    return DecoderLM(tiny_config(dtype), tp=tp, device=device).init_random(seed)


def synthetic_prompts(n: int = 4, lo: int = 16, hi: int = 64, vocab: int = 32000, seed: int = 0) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    return [torch.randint(0, vocab, (L,), generator=g).tolist() for L in lens]


def _rms(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


@torch.no_grad()
def oracle_logits(model: DecoderLM, ids: list[int]) -> torch.Tensor:
    """Logits of the last position for one sequence, fp32, no cache, no custom ops."""
    cfg = model.cfg
    Hq, Hkv, D, eps = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rms_eps
    x = model.embed_tokens.float()[torch.tensor(ids)]
    T = x.shape[0]
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D)).float()
    ang = pos[:, None] * inv[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(t):
        a, b = t[..., :D // 2], t[..., D // 2:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)

    mask = torch.full((T, T), float("-inf")).triu(1)
    for layer in model.layers:
        at = layer.self_attn
        h = _rms(x, layer.input_layernorm.float(), eps)
        qkv = F.linear(h, at.qkv_proj.float(), None if at.qkv_bias is None else at.qkv_bias.float())
        q = rot(qkv[:, :Hq * D].reshape(T, Hq, D))
        k = rot(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D))
        v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
        k = k.repeat_interleave(Hq // Hkv, 1)
        v = v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D) + mask
        a = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(T, Hq * D)
        x = x + F.linear(a, at.o_proj.float())
        h = _rms(x, layer.post_attention_layernorm.float(), eps)
        gu = F.linear(h, layer.mlp.gate_up_proj.float())
        x = x + F.linear(F.silu(gu[:, 0::2]) * gu[:, 1::2], layer.mlp.down_proj.float())
    h = _rms(x[-1], model.norm.float(), eps)
    return F.linear(h, model.head_weight().float())


@torch.no_grad()
def oracle_generate(model: DecoderLM, prompts: list[list[int]], n_tokens: int = 32) -> list[list[int]]:
    outs = []
    for p in prompts:
        ids, gen = list(p), []
        for _ in range(n_tokens):
            t = int(torch.argmax(oracle_logits(model, ids)).item())
            gen.append(t)
            ids.append(t)
        outs.append(gen)
    return outs


@torch.no_grad()
def oracle_violations(model: DecoderLM, prompts: list[list[int]], generated: list[list[int]], rel_tol: float = 2e-2):
    """Teacher-forced check of greedy generations against the fp32 oracle. At every step the oracle scores the
    prompt plus the tokens generated so far; the generated token must be the oracle's argmax, or its oracle logit
    must lie within ``rel_tol`` x (largest |logit|) of the top one (a near tie that reduced-precision arithmetic may
    resolve the other way). Returns (violations as (prompt, step, token, gap), exact-argmax fraction)."""
    bad, exact, total = [], 0, 0
    for pi, (p, gen) in enumerate(zip(prompts, generated)):
        ids = list(p)
        for step, t in enumerate(gen):
            lg = oracle_logits(model, ids)
            top = float(lg.max())
            gap = top - float(lg[int(t)])
            total += 1
            if int(torch.argmax(lg)) == int(t):
                exact += 1
            elif gap > rel_tol * float(lg.abs().max()):
                bad.append((pi, step, int(t), gap))
            ids.append(int(t))
    return bad, exact / max(1, total)


def fp32_copy(model: DecoderLM) -> DecoderLM:
    """The same weights (as stored, e.g. bf16-rounded) in an fp32 model on the CPU, for the oracle."""
    m = build_tiny(device="cpu", dtype=torch.float32)
    for (_, a), (_, b) in zip(m.named_parameters(), model.named_parameters()):
        a.copy_(b.float().cpu())
    return m
