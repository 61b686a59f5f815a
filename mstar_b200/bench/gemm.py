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
    ap.add_argument("--trace", action="store_true", help="print the phase timeline of the CTAs of one launch")
    ap.add_argument("--packed", action="store_true", help="weight stored tile by tile (gemm.pack_weight)")
    a = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = (torch.randn(a.m, a.k, device=dev, generator=g) * 0.1).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev, generator=g) * 0.1).bfloat16()
    ep = {"none": gemm.EPILOGUE_NONE, "swiglu": gemm.EPILOGUE_SWIGLU, "gelu": gemm.EPILOGUE_GELU}[a.epilogue]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    err = None
    if a.packed:
        wp = gemm.pack_weight(w)
        y0 = gemm.linear(x, w, epilogue=ep, force_splits=a.splits).float()
        y1 = gemm.linear(x, wp, epilogue=ep, force_splits=a.splits).float()
        err = (y0 - y1).abs().max().item()
        w = wp
    for _ in range(a.warmup):
        gemm.linear(x, w, epilogue=ep, force_splits=a.splits)
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        if flush is not None:
            flush.fill_(1)
            _ = flush.view(torch.int32).sum()      # a read pass after the write: the timed kernel starts on a clean L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gemm.linear(x, w, epilogue=ep, force_splits=a.splits)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    if a.trace:
        import ctypes
        from ..ops import _lib
        tr = torch.zeros(1 << 16, 8, dtype=torch.int64, device=dev)
        _lib.kernels().mstar_gemm_set_trace(ctypes.c_void_p(tr.data_ptr()))
        if flush is not None:
            flush.fill_(1)
            _ = flush.view(torch.int32).sum()
        gemm.linear(x, w, epilogue=ep, force_splits=a.splits)
        torch.cuda.synchronize()
        _lib.kernels().mstar_gemm_set_trace(ctypes.c_void_p(0))
        t = tr[tr[:, 0] > 0].cpu().double()
        t0 = t[:, 0].min()
        names = ["entry", "prologue done", "accumulator staged in shared memory", "first tile landed",
                 "last umma issued", "accumulator ready", "epilogue (or partial tile) done", "cluster slice stored"]
        rows = {}
        for i, nme in enumerate(names):
            c = t[:, i][t[:, i] > 0] - t0
            if c.numel():
                rows[nme] = [round(float(c.min()) / 1e3, 2), round(float(c.median()) / 1e3, 2),
                             round(float(c.max()) / 1e3, 2)]
        print(json.dumps({"ctas": int(t.shape[0]), "us_after_first_entry[min,median,max]": rows}))
    ts.sort()
    ms = ts[len(ts) // 2]
    flops = 2.0 * a.m * a.n * a.k
    byts = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    print(json.dumps({"m": a.m, "n": a.n, "k": a.k, "epilogue": a.epilogue, "ms": round(ms, 4),
                      "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                      "splits_forced": a.splits, "packed": a.packed, "packed_vs_plain_max_err": err,
                      "plan": gemm.gemm_plan(a.m, a.n, a.k)}))


if __name__ == "__main__":
    main()
