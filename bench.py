"""Headline benchmark: decode tokens/s per box (plus p50 TTFT) of the Orpheus-3B-class TTS backbone
(Llama-3.2-3B shape: 28 layers, hidden 3072, 24 q / 8 KV heads of 128, FFN 8192, vocabulary 156,940), bf16,
random-init weights, synthetic token ids, 64 concurrent requests per model replica.

    python bench.py --gpus N --steps K --warmup W            (N > 1 under torchrun, one rank per GPU)
    python bench.py --impl reference ...                     (the reference's own stack, if installed)

A "step" is one decode step of every running request (64 tokens per replica). Contexts are in the steady state
of 1200-token generations: each request's prompt (32-128 random ids) is followed by U(0, 1200) already generated
tokens, all of it prefilled for real before the timed region. Two numbers are produced:
  * value / ms_per_step: K replays of the captured decode step, timed with CUDA events (max over ranks);
  * e2e: K calls of the engine's public ``LLMEngine.step()`` — plan staged in pinned host memory and copied to
    the device, graph replay, sampled tokens copied back to pinned host memory and read — timed on the host
    with a device synchronize on both sides.
Weights (6.4 GB) and KV (about 5 GB) are far larger than L2, so no explicit L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s_per_box"
MODEL = "orpheus-3b-class (llama-3.2-3b backbone, vocab 156940)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler running beside the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    """The unmodified reference through its own public API. Reports ``unavailable`` when it cannot run here."""
    try:
        from baseline.reference_bench import run_reference
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference harness not importable: {e}"}))
        return
    print(json.dumps(run_reference(args)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree inside a replica (replicas = gpus / tp)")
    ap.add_argument("--concurrency", type=int, default=64, help="concurrent requests per replica")
    ap.add_argument("--gen-tokens", type=int, default=1200)
    ap.add_argument("--ttft-samples", type=int, default=8)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-serving", action="store_true",
                    help="skip the HTTP serving measurement (LLM + codec behind the C++ frontend, 1 GPU only)")
    ap.add_argument("--profile-step", action="store_true",
                    help="run ONE eager decode step between cudaProfilerStart/Stop and exit (for ncu "
                         "--profile-from-start off)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.engine.llm_engine import LLMEngine
    from mstar_b200.models.decoder import DecoderLM
    from mstar_b200.models.orpheus_config import orpheus_3b_config
    from mstar_b200.ops import _counters
    from mstar_b200.ops.sampling import SamplingConfig
    from mstar_b200.parallel.comm import CommGroup, init_from_env

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    world_group = init_from_env()
    tp = CommGroup.trivial()
    if args.tp > 1:
        from mstar_b200.parallel.symm import attach_symmetric_heap
        ranks = [r for r in range(world) if r // args.tp == rank // args.tp]
        groups = [dist.new_group([r for r in range(world) if r // args.tp == g]) for g in range(world // args.tp)]
        tp = CommGroup(groups[rank // args.tp], ranks, rank)
        attach_symmetric_heap(tp, dev)

    cfg = orpheus_3b_config()
    model = DecoderLM(cfg, tp=tp, device=dev).init_random(seed=0)
    C = args.concurrency
    ps = 128
    max_ctx = 128 + args.gen_tokens + 2 * (args.steps + max(args.warmup, 3)) + 192
    pages = C * ((max_ctx + ps - 1) // ps) + 64
    kvc = KVCacheConfig(num_layers=cfg.num_layers, num_kv_heads=max(1, cfg.num_kv_heads // tp.size),
                        head_dim=cfg.head_dim, max_seq_len=max_ctx, max_num_pages=pages, page_size=ps,
                        num_qo_heads=cfg.num_heads // tp.size)
    eng = LLMEngine(model, kvc, dev, max_batch=C, max_prefill_tokens=16384, capture_sizes=[C], track_seen=True)
    samp = SamplingConfig(cfg.vocab_size, temperature=0.6, top_p=0.8, repetition_penalty=1.3, ignore_eos=True)

    # every replica gets the same synthetic load (seeded per replica)
    g = torch.Generator().manual_seed(1234 + rank // tp.size)
    plens = torch.randint(32, 129, (C,), generator=g).tolist()
    total_new = args.steps * 2 + args.warmup * 2 + 8
    # tokens already generated when the measurement starts: drawn so that the contexts stay inside the workload's range
    # (prompt + up to gen_tokens) while the timed steps add to them
    done = torch.randint(0, max(1, args.gen_tokens - total_new), (C,), generator=g).tolist()
    for i in range(C):
        ids = torch.randint(0, cfg.vocab_size, (plens[i] + done[i],), generator=g).tolist()
        eng.add_request(f"req{rank}_{i}", ids, total_new, samp)

    # prefill everything (several packed forwards), then W warm-up decode steps through the public step()
    while eng.waiting:
        eng.step()
    for _ in range(max(args.warmup, 3)):
        eng.step()
    torch.cuda.synchronize()
    eng.check_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile_step:
        live = {i: r for i, r in enumerate(eng._rows) if r is not None}
        ctx = eng._plan_rows(live, C)
        ctx.plan.splits = eng._graph_splits.get(C, 1)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng._decode_body(ctx)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "one eager decode step", "batch": C}))
        return

    # clocks are sampled across both timed regions (end-to-end steps, then device-timed replays): same load
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)          # nvidia-smi needs a moment before its first sample
    # ---- (1) end to end through the public API ----
    e2e = None
    if not args.no_e2e:
        barrier()
        h0, d0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"]
        s0 = eng.stats["decode_steps"]
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.step()
        eng._drain()
        torch.cuda.synchronize()
        t_e2e = time.perf_counter() - t0
        nsteps = eng.stats["decode_steps"] - s0
        assert nsteps == args.steps, (nsteps, args.steps)
        e2e = dict(t=t_e2e, h2d=(eng.stats["h2d_bytes"] - h0) / nsteps, d2h=(eng.stats["d2h_bytes"] - d0) / nsteps)

    # ---- (2) device-timed replays of the captured decode step ----
    graph = eng._graphs[C]
    live = {i: r for i, r in enumerate(eng._rows) if r is not None}
    barrier()
    l0 = _counters.get()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s1 = eng.stats["decode_steps"]
    ev0.record()
    for _ in range(args.steps):
        eng.step()                       # plan upload of step n + 1 overlaps the replay of step n, as in serving
    eng._drain()
    ev1.record()
    torch.cuda.synchronize()
    assert eng.stats["decode_steps"] - s1 == args.steps
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    eng.check_status()
    launches_per_step = eng.launches_per_decode_graph.get(C, 0)

    # ---- (3) p50 TTFT: a new request entering the busy engine (prefill + first token readback) ----
    ttfts = []
    for i in range(args.ttft_samples):
        victim = next(r for r in eng._rows if r is not None)
        eng.abort(victim.request_id)
        n = int(torch.randint(32, 129, (1,), generator=g))
        ids = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        req = eng.add_request(f"ttft{rank}_{i}", ids, 64, samp)
        while req.t_first_token is None:
            eng.step(max_lag=0)
        ttfts.append((req.t_first_token - t0) * 1e3)
    ttft_p50 = statistics.median(ttfts) if ttfts else None

    # ---- reduce over ranks ----
    vals = torch.tensor([ms, e2e["t"] if e2e else 0.0, ttft_p50 or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, t_e2e, ttft_p50 = vals.tolist()
    replicas = max(1, world // tp.size)
    tokens = replicas * C * args.steps
    value = tokens / (ms / 1e3)
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform random token ids, random-init weights N(0,0.02))",
        "config": {"model": MODEL, "global_batch": replicas * C, "seq_len": "prompt 32-128 + U(0,1200) generated",
                   "parallelism": f"dp{replicas}" + (f"xtp{tp.size}" if tp.size > 1 else ""),
                   "concurrency_per_replica": C, "page_size": ps, "sampling": "temp 0.6 top_p 0.8 rep 1.3",
                   "l2": "inputs larger than L2 (6.4 GB weights + ~5 GB KV per step); no flush needed"},
        "clocks": clocks,
        "gpu_launches": int(launches_per_step * args.steps),
        "ttft_p50_ms": round(ttft_p50, 3) if ttft_p50 else None,
        "impl": "ours",
    }
    if e2e:
        out["e2e"] = {"value": round(tokens / t_e2e, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])}
    if world == 1 and not args.no_e2e and not args.no_serving:
        # the same measurement as the reference arm: the whole server (HTTP frontend, conductor, worker, LLM and
        # codec partitions on this GPU), tokens counted from the audio the clients receive
        del eng, model, graph
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            res = subprocess.run([sys.executable, "-m", "mstar_b200.bench.serve_tts", "--concurrency", str(C),
                                  "--tokens", "1204"], capture_output=True, text=True, timeout=900,
                                 cwd=os.path.dirname(os.path.abspath(__file__)))
            line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
            out["serving_http"] = json.loads(line)
        except Exception as e:  # noqa: BLE001
            out["serving_http"] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
