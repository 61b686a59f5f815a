"""Time the block-scaled fp8 GEMM on one shape against the bf16 kernel on the same shape:
``python -m mstar_b200.bench.gemm_fp8 --m 64 --n 16384 --k 3072 --flush``. The activation is quantised once outside
the timed region (its kernel is timed on its own); prints one JSON line."""
from __future__ import annotations

import argparse
import ctypes
import json

import torch

from ..ops import _lib, gemm, gemm_fp8


def _time(fn, iters, flush):
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
            _ = flush.view(torch.int32).sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = (torch.randn(a.m, a.k, device=dev, generator=g) * 0.5).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev, generator=g) * 0.05).bfloat16()
    wq = gemm_fp8.quantize_weight(w)
    q, st = gemm_fp8.quantize_act(x)
    out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
    lib = _lib.kernels()

    def run_fp8():
        rc = lib.mstar_gemm_fp8(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(st.data_ptr()), int(st.stride(0)),
                                ctypes.c_void_p(wq.data.data_ptr()), ctypes.c_void_p(wq.scale.data_ptr()),
                                ctypes.c_void_p(out.data_ptr()), a.m, a.n, a.k, a.k, a.k, a.n, None, None, 0, 0, 0,
                                ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "mstar_gemm_fp8")

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    for _ in range(a.warmup):
        run_fp8()
        gemm.linear(x, w)
        gemm_fp8.quantize_act(x)
    torch.cuda.synchronize()
    ref = gemm_fp8.linear_fp8_ref(x.cpu(), gemm_fp8.Fp8Weight(wq.data.cpu(), wq.scale.cpu())).float()
    err = (out.float().cpu() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    ms8 = _time(run_fp8, a.iters, flush)
    ms16 = _time(lambda: gemm.linear(x, w), a.iters, flush)
    msq = _time(lambda: gemm_fp8.quantize_act(x), a.iters, flush)
    flops = 2.0 * a.m * a.n * a.k
    print(json.dumps({"m": a.m, "n": a.n, "k": a.k, "fp8_ms": round(ms8, 4), "fp8_tflops": round(flops / ms8 / 1e9, 1),
                      "fp8_weight_gbs": round(a.n * a.k / ms8 / 1e6, 1), "bf16_ms": round(ms16, 4),
                      "bf16_tflops": round(flops / ms16 / 1e9, 1), "quant_act_ms": round(msq, 4),
                      "rel_err_vs_oracle": round(err, 5)}))


if __name__ == "__main__":
    main()
