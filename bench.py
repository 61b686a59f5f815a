"""Headline benchmark: decode tokens/s per box (plus p50 time to first audio) of the Orpheus-3B-class TTS deployment
(Llama-3.2-3B backbone: 28 layers, hidden 3072, 24 q / 8 KV heads of 128, FFN 8192, vocabulary 156,940; SNAC-style
24 kHz codec), bf16, random-init weights, synthetic prompts, 64 concurrent requests per GPU.

    python bench.py --gpus N --steps K --warmup W            (N > 1 under torchrun, one rank per GPU)
    python bench.py --impl reference ...                     (the reference's own stack, if installed)

Two measurements, both on the serving stack:

  * ``value`` / ``ms_per_step``: K decode steps of all 64 requests of every GPU's LLM replica, run on the SERVING
    engine (``KVCacheEngine`` with the deployment's LLM submodule) the way a worker drives it, timed with CUDA events,
    maximum over ranks. Contexts are in the steady state of 1200-token generations: every request's prompt
    (32-128 random ids) is followed by U(0, 1200) already generated tokens, all of it prefilled for real before the
    timed region. Each step's plan is uploaded from pinned host memory and its sampled ids are copied back to pinned
    host memory. Weights (6.4 GB) and KV (about 5 GB) are far larger than L2, so no explicit flush is needed.
  * ``e2e``: the whole product, as a user runs it: ONE deployment (conductor process, one worker process per GPU,
    every GPU an LLM replica and a codec replica, C++ HTTP frontend), 64 x N concurrent streaming requests of 1204
    audio tokens over ``POST /generate``, tokens counted from the audio that the clients receive, wall clock at the
    client over the window in which all requests decode. ``ttft_p50_ms`` is the p50 time to the first audio chunk
    under that load. The reference arm (``--impl reference``) is measured in exactly this way with the same client.
    Rank 0 runs it; the other ranks release their GPUs and wait.
"""
from __future__ import annotations

import argparse
import datetime
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
MODEL = "orpheus-3b-class TTS (llama-3.2-3b backbone, vocab 156940, SNAC-style 24 kHz codec)"
SEQ = "short text prompt + 1204 generated audio tokens, sliding-window codec chunks of 28 tokens"


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
        return self

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


def shared_config(n_gpus: int, concurrency: int, tp: int = 1) -> dict:
    """The part of ``config`` that both arms print identically: same model, load and placement."""
    replicas = max(1, n_gpus // tp)
    return {"model": MODEL, "global_batch": replicas * concurrency, "seq_len": SEQ,
            "parallelism": f"dp{replicas}" + (f"xtp{tp}" if tp > 1 else "")}


def reference_arm(args):
    """The unmodified reference through its own public API. Reports ``unavailable`` when it cannot run here.
    Under torchrun only rank 0 works; the other ranks leave at once (the reference spawns its own workers)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    try:
        from baseline.reference_bench import run_reference
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference harness not importable: {e}"}))
        return
    print(json.dumps(run_reference(args)), flush=True)


GENERATION_REFERENCE_UNAVAILABLE = {
    "bagel_t2i": "the reference's BAGEL server loads the published checkpoint directory (tokenizer files, ae.safetensors, "
                 "ema.safetensors, about 29 GB) at start-up; there is no network and no synthetic checkpoint of that "
                 "layout is written",
    "cosmos3_t2v": "the reference's Cosmos3 transformer imports diffusers (diffusers.models.embeddings.Timesteps), "
                   "which is not installed in this image, and there is no index to install it from",
}


def generation_workload(args) -> None:
    """Served image / video generation latency (``--workload bagel_t2i | cosmos3_t2v``): rank 0 starts the
    multi-process deployment over the GPUs of the node and times whole requests through the public API."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "workload": args.workload,
                          "unavailable": GENERATION_REFERENCE_UNAVAILABLE[args.workload]}), flush=True)
        return
    from mstar_b200.bench.serve_workloads import run_workload
    n_req = max(1, min(args.steps, 3)) if args.steps != 210 else 1
    tp, sp = (2, 2) if (args.workload == "cosmos3_t2v" and args.gpus >= 4) else ((2, 1) if args.workload == "cosmos3_t2v" and args.gpus >= 2 else (1, 1))
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))).start()
    r = run_workload(args.workload, args.gpus, requests=n_req, tp=tp, sp=sp)
    clocks = sampler.stop()
    out = {"metric": f"{args.workload} served latency", "value": r.get("value"), "unit": r["unit"], "n_gpus": args.gpus,
           "steps": n_req, "warmup": 1, "ms_per_step": None if r.get("value") is None else round(1e3 * r["value"], 1),
           "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": r["data"],
           "config": r["config"], "impl": "ours", "clocks": clocks,
           "e2e": {"value": r.get("value"), "unit": r["unit"], "timing": "wall clock from submit_request to the last "
                   "result byte, multi-process deployment", "latencies_s": r.get("latencies_s"),
                   "s_per_denoise_step": r.get("s_per_step"), "result_bytes": r.get("result_bytes")},
           "reference": GENERATION_REFERENCE_UNAVAILABLE[args.workload]}
    if "error" in r:
        out["error"] = r["error"]
    print(json.dumps(out), flush=True)


def main():
    import faulthandler
    faulthandler.enable()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=210)
    ap.add_argument("--warmup", type=int, default=14)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree inside a replica (replicas = gpus / tp)")
    ap.add_argument("--concurrency", type=int, default=64, help="concurrent requests per replica")
    ap.add_argument("--gen-tokens", type=int, default=1204)
    ap.add_argument("--no-e2e", action="store_true", help="skip the served measurement")
    ap.add_argument("--no-engine", action="store_true", help="skip the device-timed engine measurement")
    ap.add_argument("--workload", default="orpheus_tts", choices=["orpheus_tts", "bagel_t2i", "cosmos3_t2v"],
                    help="orpheus_tts is the headline; the other two are served generation latencies (one request at "
                         "a time through the multi-process deployment; --steps = timed requests)")
    args = ap.parse_args()
    if args.workload != "orpheus_tts":
        generation_workload(args)
        return
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from mstar_b200.bench.engine_decode import EngineDecodeHarness
    from mstar_b200.parallel.comm import CommGroup, init_from_env

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    init_from_env()
    host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(hours=3)) if world > 1 else None
    tp = CommGroup.trivial()
    if args.tp > 1:
        from mstar_b200.parallel.symm import attach_symmetric_heap
        ranks = [r for r in range(world) if r // args.tp == rank // args.tp]
        groups = [dist.new_group([r for r in range(world) if r // args.tp == g]) for g in range(world // args.tp)]
        tp = CommGroup(groups[rank // args.tp], ranks, rank)
        attach_symmetric_heap(tp, dev)
    C = args.concurrency
    W, K = max(args.warmup, 3), args.steps
    replicas = max(1, world // tp.size)
    out = {"metric": METRIC, "value": None, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
           "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic (uniform random token ids / short text prompts, random-init weights N(0,0.02))",
           "config": dict(shared_config(world, C, tp.size), concurrency_per_replica=C, page_size=128,
                          sampling="temp 0.6 top_p 0.8 rep 1.3", decode_burst=7,
                          l2="inputs larger than L2 (6.4 GB weights + ~5 GB KV per step); no flush needed"),
           "impl": "ours"}

    # ---- (1) device-timed steps on the serving engine ----
    if not args.no_engine:
        total_new = K + W + 16
        max_ctx = 128 + args.gen_tokens + total_new + 64
        h = EngineDecodeHarness(dev, C, max_ctx, tp_group=None if tp.is_trivial else tp)
        g = torch.Generator().manual_seed(1234 + rank // tp.size)
        plens = torch.randint(32, 129, (C,), generator=g).tolist()
        done = torch.randint(0, max(1, args.gen_tokens - total_new), (C,), generator=g).tolist()
        vocab = h.model.cfg.vocab_size
        h.prefill({f"req{rank}_{i}": torch.randint(0, vocab, (plens[i] + done[i],), generator=g).tolist()
                   for i in range(C)})
        h.decode(W)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local).start()
        time.sleep(0.3)              # nvidia-smi needs a moment before its first sample
        io0 = _io()
        ms, bursts, launches = h.decode(K)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        io1 = _io()
        clocks = sampler.stop()
        vals = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        ms = float(vals[0])
        out.update(value=round(replicas * C * K / (ms / 1e3), 1), ms_per_step=round(ms / K, 4), clocks=clocks,
                   gpu_launches=int(launches),
                   engine={"bursts": bursts, "h2d_bytes_per_step": (io1["h2d_bytes"] - io0["h2d_bytes"]) // K,
                           "d2h_bytes_per_step": (io1["d2h_bytes"] - io0["d2h_bytes"]) // K,
                           "timing": "CUDA events around K steps on the serving engine, max over ranks"})
        del h
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        # a communicating arm beside the replicas: the same engine with the model cut over PAIRS of GPUs (tensor
        # parallel 2: row-parallel partial sums reduced in the consumer norm kernels through NVLS, vocabulary cut by
        # rows), so that a run at N >= 2 also times the fused compute + collective kernels
        if world >= 2 and world % 2 == 0 and tp.is_trivial and not os.environ.get("MSTAR_BENCH_NO_TP_ARM"):
            try:
                from mstar_b200.parallel.symm import attach_symmetric_heap
                pairs = [dist.new_group([2 * g_, 2 * g_ + 1]) for g_ in range(world // 2)]
                tp2 = CommGroup(pairs[rank // 2], [rank // 2 * 2, rank // 2 * 2 + 1], rank)
                attach_symmetric_heap(tp2, dev)
                h2 = EngineDecodeHarness(dev, C, max_ctx, tp_group=tp2)
                g2 = torch.Generator().manual_seed(1234 + rank // 2)
                pl2 = torch.randint(32, 129, (C,), generator=g2).tolist()
                dn2 = torch.randint(0, max(1, args.gen_tokens - total_new), (C,), generator=g2).tolist()
                h2.prefill({f"tp{rank // 2}_{i}": torch.randint(0, vocab, (pl2[i] + dn2[i],), generator=g2).tolist()
                            for i in range(C)})
                h2.decode(W)
                torch.cuda.synchronize()
                dist.barrier()
                ms2, _, _ = h2.decode(K)
                v2 = torch.tensor([ms2], dtype=torch.float64, device=dev)
                dist.all_reduce(v2, op=dist.ReduceOp.MAX)
                out["tp2_arm"] = {"parallelism": f"dp{world // 2}xtp2", "ms_per_step": round(float(v2[0]) / K, 4),
                                  "value": round(world // 2 * C * K / (float(v2[0]) / 1e3), 1), "unit": "tokens/s",
                                  "multicast": bool(tp2.symm.mc_ptr),
                                  "kernels": "row-parallel GEMM partials summed by multimem.ld_reduce inside the "
                                             "residual + RMSNorm kernel; vocabulary-parallel embedding and head"}
                del h2
                gc.collect()
                torch.cuda.empty_cache()
            except Exception as e:  # noqa: BLE001
                out["tp2_arm"] = {"error": f"{type(e).__name__}: {e}"}

    # ---- (2) end to end through the server ----
    if not args.no_e2e:
        if host_group is not None:
            dist.barrier(group=host_group)         # every rank has released its GPU memory
        if rank == 0:
            from mstar_b200.bench.serve_tts import run_serving
            smp = ClockSampler(0).start()
            res = run_serving(world, C, args.gen_tokens, tp=tp.size)
            res["clocks_gpu0"] = smp.stop()
            workers = res.pop("workers", [])
            if "error" in res:
                out["e2e"] = {"error": res["error"]}
            else:
                steps_served = max(1, sum(e.get("decode_steps", 0) for w in workers for e in w.get("engines", [])))
                out["e2e"] = {"value": res["tokens_per_s"], "unit": "tokens/s",
                              "h2d_bytes_per_step": sum(w.get("h2d_bytes", 0) for w in workers) // steps_served,
                              "d2h_bytes_per_step": sum(w.get("d2h_bytes", 0) for w in workers) // steps_served,
                              "ms_per_step": res["ms_per_step"], "window_s": res["window_s"],
                              "ttfa_p50_ms": res["ttfa_p50_ms"], "ttfa_p99_ms": res["ttfa_p99_ms"],
                              "timing": "wall clock at the HTTP clients over the window in which all requests decode",
                              "frontend": res["frontend"], "processes": "conductor + one worker per GPU",
                              "clocks_gpu0": res["clocks_gpu0"]}
                out["ttft_p50_ms"] = res["ttfa_p50_ms"]
                dev_ms = sum(e.get("decode_device_ms", 0.0) for w in workers for e in w.get("engines", []))
                out["e2e"]["served_decode_device_ms_per_step"] = round(dev_ms / steps_served, 4)
                out["e2e"]["workers"] = [{k: w.get(k) for k in ("worker", "phase_s", "batches", "speculation")}
                                         for w in workers]
                if out["value"] is None:
                    out["value"], out["ms_per_step"] = res["tokens_per_s"], res["ms_per_step"]
        if host_group is not None:
            dist.barrier(group=host_group)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier(group=host_group)
        dist.destroy_process_group()


def _io() -> dict:
    from mstar_b200.utils import io_counters
    return io_counters.snapshot()


if __name__ == "__main__":
    main()
