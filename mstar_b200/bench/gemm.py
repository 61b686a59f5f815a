"""Time the tcgen05 GEMM on one shape: ``python -m mstar_b200.bench.gemm --m 16384 --n 9216 --k 3072``.
Prints one JSON line (CUDA-event time after warm-up, TFLOP/s, bytes moved / time for skinny shapes). Between timed
launches a buffer larger than L2 is rewritten when ``--flush`` is given (decode-shaped GEMMs re-read their weights
from HBM in real use)."""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=9216)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--epilogue", default="none", choices=["none", "swiglu", "gelu"])
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--splits", type=int, default=0, help="force the split-K factor (0 = the library's choice)")
    a = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = (torch.randn(a.m, a.k, device=dev, generator=g) * 0.1).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev, generator=g) * 0.1).bfloat16()
    ep = {"none": gemm.EPILOGUE_NONE, "swiglu": gemm.EPILOGUE_SWIGLU, "gelu": gemm.EPILOGUE_GELU}[a.epilogue]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    for _ in range(a.warmup):
        gemm.linear(x, w, epilogue=ep, force_splits=a.splits)
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gemm.linear(x, w, epilogue=ep, force_splits=a.splits)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    ms = ts[len(ts) // 2]
    flops = 2.0 * a.m * a.n * a.k
    byts = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    print(json.dumps({"m": a.m, "n": a.n, "k": a.k, "epilogue": a.epilogue, "ms": round(ms, 4),
                      "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                      "splits_forced": a.splits, "plan": gemm.gemm_plan(a.m, a.n, a.k)}))


if __name__ == "__main__":
    main()
