"""Time the sampling kernel on one shape: ``python -m mstar_b200.bench.sampling --rows 64 --vocab 156940``
(temperature 0.6, top-p 0.8, repetition penalty 1.3 over fp32 logits, as in the decode benchmark). Prints one JSON
line: CUDA-event time after warm-up, logits bytes / time."""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import sampling as S


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=156940)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--std", type=float, default=2.0, help="standard deviation of the synthetic logits")
    a = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    logits = torch.randn(a.rows, a.vocab, device=dev, generator=g) * a.std
    st = S.SamplerState(a.rows, a.vocab, dev, track_seen=True)
    for b in range(a.rows):
        st.assign(f"r{b}", S.SamplingConfig(a.vocab, temperature=0.6, top_p=0.8, repetition_penalty=1.3), seed=b + 1)
    rs = torch.arange(a.rows, dtype=torch.int32, device=dev)
    for _ in range(a.warmup):
        st.sample(logits, rs)
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st.sample(logits, rs)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    ms = ts[len(ts) // 2]
    print(json.dumps({"rows": a.rows, "vocab": a.vocab, "us": round(ms * 1e3, 1),
                      "logits_gbs": round(a.rows * a.vocab * 4 / ms / 1e6, 1)}))


if __name__ == "__main__":
    main()
