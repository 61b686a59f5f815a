"""Time one denoising forward of the two DiT styles at production shapes on one GPU (random weights, synthetic
latents): ``python -m mstar_b200.bench.dit_step --model wan22 --height 480 --width 832 --frames 81``.

Prints one JSON line: ms per forward (CUDA events, after warm-up), achieved bf16 TFLOP/s from the analytic FLOP
count, and the kernel launches per forward.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import _counters


def wan_flops(cfg, S: int, L: int, B: int) -> float:
    H, F = cfg.hidden_size, cfg.ffn_dim
    per_tok = 2 * (4 * H * H + 2 * H * H + 2 * H * F)                    # self qkv+o, cross q+o, mlp
    attn = 4 * S * H + 4 * L * H                                           # QK^T and PV, self + cross
    return B * cfg.num_layers * (S * (per_tok + attn) + 2 * L * 2 * H * H * 0)


def mot_flops(cfg, S: int, L: int, B: int) -> float:
    H, F, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    qkv = (cfg.num_heads + 2 * cfg.num_kv_heads) * D
    per_tok = 2 * (H * qkv + cfg.num_heads * D * H + 3 * H * F)
    attn = 4 * (S + L) * cfg.num_heads * D
    return B * cfg.num_layers * S * (per_tok + attn)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="wan22", choices=["wan22", "cosmos3"])
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--branches", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda")
    B = a.branches
    if a.model == "wan22":
        from ..models.dit import AdaLNDiT, wan22_5b_config
        cfg = wan22_5b_config()
        if a.layers:
            cfg.num_layers = a.layers
        m = AdaLNDiT(cfg, dev).init_random(0)
        Fl, Hl, Wl = (a.frames - 1) // 4 + 1, a.height // 16, a.width // 16
        lat = torch.randn(B, cfg.in_channels, Fl, Hl, Wl, device=dev)
        text = torch.randn(B * cfg.text_len, cfg.text_dim, device=dev, dtype=torch.bfloat16)
        kv = m.encode_context(text)
        ts = torch.full((B,), 500.0, device=dev)
        S = Fl * (Hl // 2) * (Wl // 2)
        fn = lambda: m(lat, ts, kv, [cfg.text_len] * B)  # noqa: E731
        flops = wan_flops(cfg, S, cfg.text_len, B)
    else:
        from ..engine.cache_manager import BatchedCacheManager
        from ..engine.kv_store import KVCacheConfig
        from ..models.cosmos3 import Cosmos3Transformer, cosmos3_nano_config
        from ..models.dit import grid_positions
        cfg = cosmos3_nano_config()
        if a.layers:
            cfg.num_layers = a.layers
        m = Cosmos3Transformer(cfg, 16, device=dev).init_random(0)
        L = 512
        kvc = KVCacheConfig(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, max_seq_len=1024, max_num_pages=16,
                            page_size=128, num_qo_heads=cfg.num_heads, dtype=torch.bfloat16)
        cm = BatchedCacheManager(kvc, dev, max_batch=4, max_tokens=1 << 18, n_pos_axes=3)
        G = cfg.num_heads // cfg.num_kv_heads
        ids = torch.randint(0, 1000, (L * B,), device=dev)
        ctx = cm.plan(["r"] * B, [L] * B, labels=["main", "uncond"][:B], causal=True, group=G)
        m.und.forward_hidden(m.und.embed(ids), ctx)
        cm.advance_seq_lens(ctx)
        Fl, Hl, Wl = (a.frames - 1) // 4 + 1, a.height // 8, a.width // 8
        S = Fl * (Hl // 2) * (Wl // 2)
        tok = torch.randn(S, cfg.hidden_size, device=dev, dtype=torch.bfloat16) * 0.1
        pos = grid_positions(Fl, Hl // 2, Wl // 2, dev, (L, L, L))
        gctx = cm.plan(["r"] * B, [S] * B, labels=["main", "uncond"][:B], causal=False, write_cache=False, group=G)
        fn = lambda: m.denoise(tok, pos, 500.0, B, gctx, m.proj_out_w, m.proj_out_b)  # noqa: E731
        flops = mot_flops(cfg, S, L, B)
    with torch.no_grad():
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        n0 = _counters.get()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print(json.dumps({"model": a.model, "tokens_per_branch": S, "branches": B, "layers": cfg.num_layers,
                      "ms_per_forward": round(ms, 3), "tflops": round(flops / ms / 1e9, 1),
                      "launches_per_forward": (_counters.get() - n0) // a.iters}))


if __name__ == "__main__":
    main()
