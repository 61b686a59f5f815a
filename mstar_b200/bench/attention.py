"""Time the attention kernels on one shape.
  dense (DiT / prefill):  ``python -m mstar_b200.bench.attention --mode dense --seq 8192 --heads 24 --kv-heads 24``
  decode (paged):         ``python -m mstar_b200.bench.attention --mode decode --batch 64 --ctx 2048 --heads 24 --kv-heads 8``
Prints one JSON line: CUDA-event time after warm-up, TFLOP/s (dense) or KV bytes / time (decode)."""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import attention as A


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="dense", choices=["dense", "decode"])
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv-heads", type=int, default=24)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    Hq, Hkv, D = a.heads, a.kv_heads, a.dim
    G = Hq // Hkv
    if a.mode == "dense":
        S, B = a.seq, a.batch
        q = torch.randn(B * S, Hq, D, device=dev, generator=g).bfloat16()
        k = torch.randn(B * S, Hkv, D, device=dev, generator=g).bfloat16()
        v = torch.randn(B * S, Hkv, D, device=dev, generator=g).bfloat16()
        plan = A.dense_plan([S] * B, [S] * B, G, dev, causal=a.causal)
        fn = lambda: A.attention(q, plan, k=k, v=v)  # noqa: E731
        work = 4.0 * B * S * S * Hq * D * (0.5 if a.causal else 1.0)
    else:
        B, ps = a.batch, 128
        pages_per = (a.ctx + ps - 1) // ps
        cache = (torch.randn(B * pages_per, 2, Hkv, ps, D, device=dev, generator=g) * 0.5).bfloat16()
        q = torch.randn(B, Hq, D, device=dev, generator=g).bfloat16()
        splits = A.choose_splits(B, Hkv, B, a.ctx, sm_count=3 * 148)
        plan = A.AttnPlan(q_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev),
                          kv_lens=torch.full((B,), a.ctx, dtype=torch.int32, device=dev), batch=B, num_q_tokens=B,
                          num_q_tiles=B, page_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per,
                          page_indices=torch.arange(B * pages_per, dtype=torch.int32, device=dev), splits=splits,
                          causal=True, max_q_len=1)
        fn = lambda: A.attention(q, plan, kv_cache=cache)  # noqa: E731
        work = 2.0 * B * a.ctx * Hkv * D * 2          # K and V bytes read
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    ms = ts[len(ts) // 2]
    out = {"mode": a.mode, "ms": round(ms, 4), "heads": Hq, "kv_heads": Hkv, "dim": D}
    if a.mode == "dense":
        out.update(seq=a.seq, batch=a.batch, causal=a.causal, tflops=round(work / ms / 1e9, 1))
    else:
        out.update(batch=a.batch, ctx=a.ctx, kv_gbs=round(work / ms / 1e6, 1))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
