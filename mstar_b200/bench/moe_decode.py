"""Decode throughput of a Qwen3-Omni-30B-A3B-class thinker (48 layers, hidden 2048, 32 q / 4 KV heads, 128 experts
top-8 with expert width 768, vocabulary 151936) on one GPU, bf16 experts or block-scaled fp8 experts:

    python -m mstar_b200.bench.moe_decode --requests 256 --prompt 512 --steps 64 [--fp8]

Random-init weights drawn on the device, uniform random prompt ids. The requests are prefilled through the engine's
public ``step()``; then ``--steps`` decode steps are timed with CUDA events around ``step()`` calls (plan upload,
graph replay and token read-back included). Prints one JSON line."""
from __future__ import annotations

import argparse
import dataclasses
import json
import time

import torch


@torch.no_grad()
def init_on_device(model, seed: int = 0, std: float = 0.02) -> None:
    g = torch.Generator(device=next(model.parameters()).device).manual_seed(seed)
    for name, p in model.named_parameters():
        if p.dim() >= 2:
            p.normal_(0.0, std, generator=g)
        elif "norm" in name:
            p.fill_(1.0)
        else:
            p.zero_()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=0, help="cut the layer count (0 = all 48)")
    ap.add_argument("--fp8", action="store_true")
    a = ap.parse_args()

    from ..engine.kv_store import KVCacheConfig
    from ..engine.llm_engine import LLMEngine
    from ..models.decoder import DecoderLM
    from ..models.qwen3_omni import thinker_config
    from ..ops.sampling import SamplingConfig

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = dataclasses.replace(thinker_config(torch.bfloat16), mrope_sections=None)
    if a.layers:
        cfg = dataclasses.replace(cfg, num_layers=a.layers)
    model = DecoderLM(cfg, device=dev)
    init_on_device(model)
    if a.fp8:
        model.quantize_moe_fp8()
    C, ps = a.requests, 128
    total_new = a.steps + a.warmup + 8
    max_ctx = a.prompt + total_new + 64
    pages = C * ((max_ctx + ps - 1) // ps) + 64
    kvc = KVCacheConfig(num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                        max_seq_len=max_ctx, max_num_pages=pages, page_size=ps, num_qo_heads=cfg.num_heads)
    eng = LLMEngine(model, kvc, dev, max_batch=C, max_prefill_tokens=16384, capture_sizes=[C], track_seen=False)
    samp = SamplingConfig(cfg.vocab_size, temperature=0.7, top_p=0.9, ignore_eos=True)
    g = torch.Generator().manual_seed(7)
    t0 = time.perf_counter()
    for i in range(C):
        eng.add_request(f"r{i}", torch.randint(0, cfg.vocab_size, (a.prompt,), generator=g).tolist(), total_new, samp)
    while eng.waiting:
        eng.step()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    for _ in range(max(a.warmup, 3)):
        eng.step()
    eng._drain()
    torch.cuda.synchronize()
    s0 = eng.stats["decode_steps"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.step()
    eng._drain()
    e1.record()
    torch.cuda.synchronize()
    n = eng.stats["decode_steps"] - s0
    ms = e0.elapsed_time(e1)
    eng.check_status()
    print(json.dumps({"model": "qwen3-omni-30b-a3b-class thinker", "experts": "fp8 e4m3 block-scaled" if a.fp8 else "bf16",
                      "layers": cfg.num_layers, "requests": C, "prompt_tokens": a.prompt, "decode_steps": n,
                      "ms_per_step": round(ms / n, 3), "decode_tokens_per_s": round(C * n / (ms / 1e3), 1),
                      "prefill_tokens_per_s": round(C * a.prompt / t_prefill, 1),
                      "launches_per_step": eng.launches_per_decode_graph.get(C, 0)}))


if __name__ == "__main__":
    main()
