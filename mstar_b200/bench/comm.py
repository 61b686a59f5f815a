"""Fused compute + collective kernels over the symmetric NVLink heap, each timed against the NCCL form of the same
step and against its roofline (the slower of FLOPs at the measured GEMM peak and bytes over one NVLink direction).

Run one process per GPU:

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 2 \
        -m mstar_b200.bench.comm

Every figure is a CUDA-event time around a captured graph of back-to-back calls, after warm-up, the maximum over
ranks; operands that would otherwise stay in the L2 rotate through more memory than it holds. Rank 0 prints one JSON
line per path.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer copy, one direction, per GPU
GEMM_TFLOPS = 1590.0      # measured cuBLAS bf16 burst


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        p = json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))
        return float(p.get("bf16_tflops", GEMM_TFLOPS)), float(p.get("hbm_gbs", 6650.0))
    except Exception:  # noqa: BLE001
        return GEMM_TFLOPS, 6650.0


def timed(fn, iters, warmup, dev, capture=True):
    """Device time of one call: ``iters`` calls are captured in one CUDA graph and replayed between two events, so
    neither the host's launch cost nor the skew between the ranks' hosts is in the figure (a rank that arrives early
    only waits once, at the first call). ``fn`` takes the call index, for operands that rotate through more memory
    than the L2 holds. Falls back to back-to-back eager launches when the capture fails."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    graph = None
    try:
        if not capture:
            raise RuntimeError("eager timing requested")
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                for i in range(iters):
                    fn(i)
        torch.cuda.current_stream().wait_stream(s)
        graph = g
    except Exception:  # noqa: BLE001
        torch.cuda.synchronize()
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    use_graph = bool(ok.item())
    best = None
    for _ in range(3):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if use_graph:
            graph.replay()
        else:
            for i in range(iters):
                fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / iters
        best = t if best is None else min(best, t)
    t = torch.tensor([best], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3          # microseconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=84480, help="sequence length of the Ulysses exchange")
    args = ap.parse_args()

    from ..ops import _lib, gemm
    from ..ops.elementwise import cfg_combine
    from ..parallel.comm import init_from_env
    from ..parallel.symm import attach_symmetric_heap

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    g = init_from_env()
    W, R = g.size, g.rank
    heap = attach_symmetric_heap(g, dev, slot_bytes=64 << 20, user_bytes=768 << 20)
    tflops, _ = _peaks()
    rows = []

    def report(**kw):
        rows.append(kw)
        if R == 0:
            print(json.dumps(kw), flush=True)

    # ---- decode all-reduce (64 x 3072 bf16), latency bound ----
    x = torch.randn(64, 3072, device=dev).to(torch.bfloat16)
    res = torch.randn(64, 3072, device=dev).to(torch.bfloat16)
    out = torch.empty_like(x)
    t_ours = timed(lambda i: heap.all_reduce(x, residual=res, out=out), args.iters, args.warmup, dev)
    y = x.clone()

    def nccl_ar(i):
        y.copy_(x)
        dist.all_reduce(y)
        y.add_(res)
    t_nccl = timed(nccl_ar, args.iters, args.warmup, dev)
    t_nvls = timed(lambda i: heap.all_reduce_nvls(x, residual=res, out=out), args.iters, args.warmup, dev)
    report(path="all-reduce + residual, 64x3072 bf16", ranks=W, push_us=round(t_ours, 2), nvls_us=round(t_nvls, 2),
           nccl_us=round(t_nccl, 2), multicast=bool(heap.mc_ptr))

    # ---- DiT-sized all-reduce (the tokens of one sequence-parallel rank x hidden), bandwidth bound ----
    xb = torch.randn(21120, 2048, device=dev).to(torch.bfloat16)
    ob = torch.empty_like(xb)
    t_ours = timed(lambda i: heap.all_reduce(xb, out=ob), args.iters, args.warmup, dev)
    yb = xb.clone()
    t_nccl = timed(lambda i: dist.all_reduce(yb), args.iters, args.warmup, dev)
    link_us = 2 * (W - 1) / W * xb.numel() * 2 / (LINK_GBS * 1e3)
    t_nvls = timed(lambda i: heap.all_reduce_nvls(xb, out=ob), args.iters, args.warmup, dev)
    # in-switch reduction: a rank pulls its 1/W share reduced and multicasts it: N/W in and N/W out per GPU... the
    # slower direction carries (W - 1) / W of the message once
    nvls_link_us = (W - 1) / W * xb.numel() * 2 / (LINK_GBS * 1e3)
    # the same message already resident in a symmetric region (where a row-parallel GEMM writes it): in-place
    big = heap.new_region(2 * xb.numel() * 2 + (1 << 20))        # the tensor, and staging room for the fused GEMM
    boff = big.alloc(xb.numel() * 2)
    big.view(boff, xb.shape, torch.bfloat16).zero_()
    t_inpl = timed(lambda i: heap.all_reduce_inplace(big, boff, xb.numel()), args.iters, args.warmup, dev)
    report(path="all-reduce, 21120x2048 bf16", ranks=W, push_us=round(t_ours, 2), nvls_us=round(t_nvls, 2),
           nvls_inplace_us=round(t_inpl, 2), nccl_us=round(t_nccl, 2), roofline_us=round(nvls_link_us, 2),
           frac_of_roofline=round(nvls_link_us / min(t_ours, t_nvls, t_inpl), 3), multicast=bool(heap.mc_ptr))
    # large row-parallel projection (a DiT block's output projection over one rank's tokens): the GEMM writes its
    # partial into the region and the in-place all-reduce follows, against GEMM + NCCL all-reduce
    Mb, Nb, Kb = 21120, 2048, 2048 // W
    xg = torch.randn(Mb, Kb, device=dev).to(torch.bfloat16)
    wg = (torch.randn(Nb, Kb, device=dev) * 0.02).to(torch.bfloat16)
    yv = big.view(boff, (Mb, Nb), torch.bfloat16)

    def gemm_inplace(i):
        gemm.linear(xg, wg, out=yv)
        heap.all_reduce_inplace(big, boff, Mb * Nb)

    def gemm_nccl(i):
        dist.all_reduce(gemm.linear(xg, wg))
    t_gi = timed(gemm_inplace, args.iters, args.warmup, dev)
    t_gn = timed(gemm_nccl, args.iters, args.warmup, dev)
    tiles = {}
    for nc in (16, 24, 32):
        tiles[nc] = timed(lambda i: heap.linear_all_reduce_tiles(xg, wg, big, boff, n_comm=nc), args.iters, args.warmup, dev)
    best_nc = min(tiles, key=tiles.get)
    t_g0 = timed(lambda i: gemm.linear(xg, wg, out=yv), args.iters, args.warmup, dev)
    report(path=f"GEMM with the all-reduce inside, row groups overlapped ({Mb}x{Nb}x{Kb} per rank)", ranks=W,
           fused_us=round(tiles[best_nc], 2), comm_ctas=best_nc, by_comm_ctas={k: round(v, 2) for k, v in tiles.items()},
           gemm_plus_nccl_us=round(t_gn, 2), gemm_alone_us=round(t_g0, 2),
           roofline_us=round(max(nvls_link_us, 2.0 * Mb * Nb * Kb / (tflops * 1e6)), 2),
           frac_of_roofline=round(max(nvls_link_us, 2.0 * Mb * Nb * Kb / (tflops * 1e6)) / tiles[best_nc], 3))
    report(path=f"GEMM -> in-place all-reduce ({Mb}x{Nb}x{Kb} per rank)", ranks=W, fused_us=round(t_gi, 2),
           gemm_plus_nccl_us=round(t_gn, 2), gemm_alone_us=round(t_g0, 2),
           roofline_us=round(max(nvls_link_us, 2.0 * Mb * Nb * Kb / (tflops * 1e6)), 2), multicast=bool(big.mc_ptr))
    del big

    # ---- row-parallel projection: GEMM with the all-reduce in its epilogue (o_proj / down_proj of a decode step) ----
    for (M, N, K, name) in [(64, 3072, 3072 // W, "o_proj"), (64, 3072, 8192 // W, "down_proj")]:
        xa = torch.randn(M, K, device=dev).to(torch.bfloat16)
        nw = max(2, (192 << 20) // (N * K * 2) + 1)          # weight copies: together larger than the L2
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(nw)]
        r2 = torch.randn(M, N, device=dev).to(torch.bfloat16)
        t_f = timed(lambda i: heap.linear_all_reduce(xa, ws[i % nw], residual=r2), args.iters, args.warmup, dev)

        def base(i):
            yy = gemm.linear(xa, ws[i % nw])
            dist.all_reduce(yy)
            yy.add_(r2)
        t_b = timed(base, args.iters, args.warmup, dev)
        t_g = timed(lambda i: gemm.linear(xa, ws[i % nw], residual=r2), args.iters, args.warmup, dev)
        # roofline: the weight stream from HBM (N*K*2 bytes) against the partial tiles crossing NVLink
        link_us = M * N * 2 * (W - 1) / (LINK_GBS * 1e3)
        hbm_us = N * K * 2 / (_peaks()[1] * 1e3)
        report(path=f"GEMM -> all-reduce fused ({name} {M}x{N}x{K} per rank)", ranks=W, fused_us=round(t_f, 2),
               gemm_plus_nccl_us=round(t_b, 2), gemm_alone_us=round(t_g, 2),
               roofline_us=round(max(link_us, hbm_us), 2), frac_of_roofline=round(max(link_us, hbm_us) / t_f, 3))

    # ---- row-parallel projection whose reduction is done by the consumer: the GEMM writes its partial into a heap
    # slot, the residual-add + RMSNorm kernel that follows reads every row as a sum over the ranks' slots (in the
    # switch). Baseline: GEMM, NCCL all-reduce, fused add + norm kernel. ----
    from ..ops import norm as norm_ops
    from ..parallel.tp_fused import TPFusedContext
    tpf = TPFusedContext(heap, 3072, 16384)
    gamma = torch.ones(3072, device=dev, dtype=torch.bfloat16)
    for (M, N, K, name) in [(64, 3072, 3072 // W, "o_proj"), (64, 3072, 8192 // W, "down_proj"),
                            (8192, 3072, 8192 // W, "down_proj prefill")]:
        xa = torch.randn(M, K, device=dev).to(torch.bfloat16)
        nw = max(2, (192 << 20) // (N * K * 2) + 1)
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(nw)]
        r2 = torch.randn(M, N, device=dev).to(torch.bfloat16)
        r2s = tpf.residual_rows(r2).contiguous()        # large M: the residual stream is cut by rows

        def fused_rrn(i):
            gemm.linear(xa, ws[i % nw], out=tpf.partial_out(i & 1, M))
            tpf.reduce_norm(i & 1, M, gamma, 1e-5, r2s)

        def base_rrn(i):
            yy = gemm.linear(xa, ws[i % nw])
            dist.all_reduce(yy)
            norm_ops.norm(yy, gamma, 1e-5, residual=r2)

        def alone(i):
            yy = gemm.linear(xa, ws[i % nw])
            norm_ops.norm(yy, gamma, 1e-5, residual=r2)
        t_f = timed(fused_rrn, args.iters, args.warmup, dev)
        t_b = timed(base_rrn, args.iters, args.warmup, dev)
        t_1 = timed(alone, args.iters, args.warmup, dev)
        link_us = M * N * 2 * (W - 1) / W / (LINK_GBS * 1e3)
        hbm_us = N * K * 2 / (_peaks()[1] * 1e3)
        flop_us = 2.0 * M * N * K / (tflops * 1e6)
        roof = max(link_us, hbm_us, flop_us)
        report(path=f"GEMM -> reduce in the consumer norm ({name} {M}x{N}x{K} per rank)", ranks=W,
               fused_us=round(t_f, 2), gemm_nccl_norm_us=round(t_b, 2), gemm_norm_no_comm_us=round(t_1, 2),
               roofline_us=round(roof, 2), frac_of_roofline=round(roof / t_f, 3), multicast=bool(tpf.region.mc_ptr))

    # ---- vocabulary-parallel head: logits shard GEMM + multicast all-gather vs the full head on every rank ----
    V = 156940
    tpv = TPFusedContext(heap, 3072, 64, vocab=V, max_logit_rows=64)
    hrows = torch.randn(64, 3072, device=dev).to(torch.bfloat16)
    w_sh = (torch.randn(tpv.rows_per_rank, 3072, device=dev) * 0.02).to(torch.bfloat16)
    w_full = (torch.randn(V, 3072, device=dev) * 0.02).to(torch.bfloat16)
    t_vp = timed(lambda i: tpv.logits(hrows, w_sh), args.iters, args.warmup, dev)
    t_full = timed(lambda i: gemm.linear(hrows, w_full), args.iters, args.warmup, dev)
    hbm_us = tpv.rows_per_rank * 3072 * 2 / (_peaks()[1] * 1e3)
    link_us = 64 * tpv.rows_per_rank * 2 * (W - 1) / (LINK_GBS * 1e3)
    report(path=f"vocabulary-parallel head 64x{V}x3072: shard GEMM + multicast all-gather", ranks=W,
           fused_us=round(t_vp, 2), replicated_head_us=round(t_full, 2), roofline_us=round(max(hbm_us, link_us), 2),
           frac_of_roofline=round(max(hbm_us, link_us) / t_vp, 3))
    del w_full

    # ---- Ulysses head <-> sequence exchange by peer stores ----
    H, D = 8, 128          # the heads of one tensor-parallel rank (16 heads, tp 2)
    S = args.tokens // W * W
    seq_off = [S // W * i for i in range(W + 1)]
    mine = torch.randn(S // W, H, D, device=dev).to(torch.bfloat16)
    off_f = heap.alloc_user(S * (H // W) * D * 2)
    t_a2a = timed(lambda i: heap.a2a_heads(mine, off_f, True, H, D, seq_off), args.iters, args.warmup, dev)
    src = mine.view(S // W, W, H // W, D).permute(1, 0, 2, 3).contiguous()
    dst = torch.empty_like(src)

    def nccl_a2a(i):
        s2 = mine.view(S // W, W, H // W, D).permute(1, 0, 2, 3).contiguous()
        dist.all_to_all_single(dst, s2)
    t_na = timed(nccl_a2a, args.iters, args.warmup, dev)
    link_us = mine.numel() * 2 * (W - 1) / W / (LINK_GBS * 1e3)
    report(path=f"Ulysses exchange, {S} tokens x {H} heads x {D}", ranks=W, ours_us=round(t_a2a, 2),
           nccl_us=round(t_na, 2), roofline_us=round(link_us, 2), frac_of_roofline=round(link_us / t_a2a, 3),
           gbs_out_per_rank=round(mine.numel() * 2 * (W - 1) / W / t_a2a / 1e3, 1))

    # ---- QK-norm + RoPE whose stores are the head scatter, against the RoPE kernel + three exchange kernels ----
    from ..ops import rope as rope_ops
    from ..parallel.comm import CommGroup
    from ..parallel.sequence_parallel import UlyssesExchange
    Hq_, Hkv_, Sx = 16, 4, (args.tokens // 2) // W * W          # one tensor-parallel shard of 32 / 8 heads, sp = W
    try:
        spg = CommGroup(dist.group.WORLD, list(range(W)), R)
        spg.symm = heap
        ex = UlyssesExchange(spg, Sx, Hq_, Hkv_, D)
        Tl = ex.off[R + 1] - ex.off[R]
        qkv_l = torch.randn(Tl, (Hq_ + 2 * Hkv_) * D, device=dev).to(torch.bfloat16)
        pos_l = torch.randint(0, 4096, (3, Tl), device=dev, dtype=torch.int32)
        inv_f = (1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev).float() / D)))
        axis = (torch.arange(D // 2, device=dev) % 3).to(torch.int8)
        gq = torch.ones(D, device=dev, dtype=torch.bfloat16)

        def separate(i):
            q0, k0, v0 = rope_ops.rope_kv(qkv_l, pos_l, inv_f, Hq_, Hkv_, D, axis_of_freq=axis, q_norm_w=gq, k_norm_w=gq,
                                          norm_eps=1e-6, dense_kv=True)
            ex.to_heads(q0, k0, v0)
        t_sep = timed(separate, args.iters, args.warmup, dev)
        t_fus = timed(lambda i: ex.rope_to_heads(qkv_l, pos_l, inv_f, axis, gq, gq, 1e-6), args.iters, args.warmup, dev)
        out_bytes = Tl * (Hq_ + 2 * Hkv_) * D * 2 * (W - 1) / W
        report(path=f"QK-norm + RoPE + Ulysses head scatter in one kernel, {Sx} tokens x ({Hq_}+2x{Hkv_}) heads x {D}",
               ranks=W, fused_us=round(t_fus, 2), rope_then_three_exchanges_us=round(t_sep, 2),
               roofline_us=round(out_bytes / (LINK_GBS * 1e3), 2),
               frac_of_roofline=round(out_bytes / (LINK_GBS * 1e3) / t_fus, 3))
    except MemoryError:
        report(path="QK-norm + RoPE + Ulysses head scatter", skipped="symmetric heap user region too small")

    # ---- CFG-parallel gather fused with the guidance combine + Euler step (rank 0 combines) ----
    rws, cols = 4096, 64 * 16          # a 1024x1024 image: 4096 latent tokens x (2x2x16) channels, fp32 velocities
    v_off = heap.alloc_user(rws * cols * 4)
    heap.local_view(v_off, (rws, cols), torch.float32).normal_()
    xx = torch.randn(rws, cols, device=dev)
    heap.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    if R == 0:
        def fused(i):
            heap.cfg_combine(v_off, 0, 1, -1, xx, dt=-0.02, s_text=4.0, renorm=True, wait_peers=False)
    else:
        def fused(i):
            pass
    t_c = timed(fused, args.iters, args.warmup, dev)
    vu = torch.empty(rws, cols, device=dev)
    vl = heap.local_view(v_off, (rws, cols), torch.float32)

    def base_cfg(i):
        if R == 1:
            dist.send(vl, 0)
        elif R == 0:
            dist.recv(vu, 1)
            cfg_combine(vl, vu, xx, -0.02, 4.0, renorm=True)
    t_cb = timed(base_cfg, args.iters, args.warmup, dev, capture=False)     # NCCL send / recv: eager launches
    link_us = rws * cols * 4 / (LINK_GBS * 1e3)
    report(path=f"CFG gather + combine + Euler step, {rws}x{cols} fp32", ranks=W, fused_us=round(t_c, 2),
           nccl_recv_plus_combine_us=round(t_cb, 2), roofline_us=round(link_us, 2),
           frac_of_roofline=round(link_us / t_c, 3))

    torch.cuda.synchronize()
    code = _lib.read_status(clear=True)[0]
    if R == 0:
        print(json.dumps({"status_word": int(code)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
