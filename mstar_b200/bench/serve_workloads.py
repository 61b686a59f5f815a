"""Served latency of the image / video generation workloads through the public server API: BAGEL-7B-MoT-class
text-to-image (1024 x 1024, 50 flow steps, packed 2-branch guidance on one GPU; guidance branches on their own GPUs
with ``--gpus 3``) and Cosmos3-Nano-class text-to-video (480p x 93 frames by default, 35 steps, guidance 6; ``dit``
tensor- / sequence-parallel over the GPUs given). The deployment is the multi-process one (conductor process, one
worker process per GPU); a request is submitted with ``APIServer.submit_request`` and timed on the wall clock from
submission to the last byte of the encoded result, so prompt preprocessing, every denoise step's scheduling, the VAE
decode and the PNG / video encoding are all inside the number. Weights are random-init of the published shapes.

    python -m mstar_b200.bench.serve_workloads --workload bagel_t2i [--gpus 1|3]
    python -m mstar_b200.bench.serve_workloads --workload cosmos3_t2v [--gpus 1|2|4] [--tp 2 --sp 2]

Reference counterparts: benchmark/cosmos3/video_bench.py, bench_t2i_oai.py (latency per request at concurrency 1),
benchmark/runner.py.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time


def bagel_config(n_gpus: int) -> tuple[dict, dict]:
    groups = [{"node_names": ["vit_encoder", "vae_encoder", "LLM", "vae_decoder"], "ranks": [0]}]
    kw = dict(height=1024, width=1024, num_steps=50, cfg_text_scale=4.0, seed=0)
    if n_gpus >= 3:         # guidance branches on their own GPUs, combined by the fused gather + combine kernel
        groups += [{"node_names": ["LLM_cfg_text"], "ranks": [1]}, {"node_names": ["LLM_cfg_img", "combine_cfg"], "ranks": [2]}]
        kw["cfg_parallel"] = True
    return {"model": "bagel", "model_kwargs": {}, "node_groups": groups, "max_batch_size": 8}, kw


def cosmos3_config(n_gpus: int, tp: int, sp: int, height: int, width: int, frames: int) -> tuple[dict, dict]:
    ranks = list(range(max(1, tp * sp)))
    dit = {"node_names": ["dit"], "ranks": ranks}
    if tp > 1:
        dit["tp_size"] = tp
    if sp > 1:
        dit["sp_size"] = sp
    side = {"node_names": ["vae_encoder", "vae_decoder", "audio_decoder"], "ranks": [min(n_gpus - 1, ranks[-1])]}
    tokens = ((frames - 1) // 4 + 1) * (height // 16) * (width // 16)
    pages = 64
    cfg = {"model": "cosmos3", "model_kwargs": {"page_size": 128, "max_num_pages": pages}, "node_groups": [dit, side],
           "max_batch_size": 8}
    kw = dict(height=height, width=width, num_frames=frames, num_steps=35, guidance_scale=6.0, seed=0,
              negative_prompt="blurry, low quality")
    return cfg, dict(kw, _tokens=tokens)


def run_workload(workload: str, n_gpus: int = 1, *, requests: int = 1, warm_steps: int = 2, tp: int = 1, sp: int = 1,
                 height: int = 480, width: int = 832, frames: int = 93, steps: int | None = None,
                 small: bool = False) -> dict:
    """``small``: test-sized weights and a 32 x 32 frame (CPU smoke run of the same code path)."""
    from ..api_server.server import APIServer
    if workload == "bagel_t2i":
        cfg, kw = bagel_config(n_gpus)
        outs, unit, prompt = ["image"], "s/image", "A photograph of a lighthouse on a cliff at dawn, waves below"
        desc = {"model": "BAGEL-7B-MoT-class (28 layers, hidden 3584, understanding + generation experts)",
                "resolution": "1024x1024", "steps": 50, "cfg_text_scale": 4.0,
                "parallelism": "cfg-parallel x3" if n_gpus >= 3 else "1 GPU, guidance branches packed"}
    elif workload == "cosmos3_t2v":
        cfg, kw = cosmos3_config(n_gpus, tp, sp, height, width, frames)
        tokens = kw.pop("_tokens")
        outs, unit, prompt = ["video"], "s/video", "A robot arm stacks three wooden blocks on a table"
        desc = {"model": "Cosmos3-Nano-class (36 layers, hidden 4096, 32/8 heads, dual pathway)",
                "resolution": f"{width}x{height}x{frames}", "latent_tokens": tokens, "steps": 35, "guidance": 6.0,
                "parallelism": f"tp{tp}xsp{sp}" if tp * sp > 1 else "1 GPU, guidance branches packed"}
    else:
        raise ValueError(workload)
    if small:
        cfg["model_kwargs"] = dict(cfg["model_kwargs"], small=True, **({"page_size": 16} if workload == "cosmos3_t2v" else {}))
        kw.update(height=32, width=32, num_steps=3, **({"num_frames": 5} if workload == "cosmos3_t2v" else {}))
        desc = dict(desc, model=desc["model"] + " [test-sized]", resolution="32x32", steps=3)
    if steps:
        kw["num_steps"] = steps
        desc["steps"] = steps
    out = {"bench": "serve_workloads", "workload": workload, "n_gpus": n_gpus, "unit": unit, "config": desc,
           "data": "synthetic (short text prompt, random-init weights of the published shapes)"}
    if tp * sp > 1:
        # seconds-long steps on a mesh: the ranks' first steps differ by more than the 2 s default of the device waits
        import os
        os.environ.setdefault("MSTAR_WAIT_LIMIT_MS", "60000")
    srv = APIServer(cfg, in_process=False).start(3600)
    try:
        # warm-up: the same request with a few steps (kernel attributes, graph capture of the step, allocator pools)
        t0 = time.time()
        rid = srv.submit_request(prompt, output_modalities=outs, model_kwargs=dict(kw, num_steps=warm_steps))
        res = srv.collect_results(rid, 3600)
        if "error" in res:
            raise RuntimeError(res["error"][0].data.decode(errors="replace"))
        out["warmup_s"] = round(time.time() - t0, 2)
        lat, sizes = [], []
        for _ in range(requests):
            t0 = time.time()
            rid = srv.submit_request(prompt, output_modalities=outs, model_kwargs=dict(kw))
            res = srv.collect_results(rid, 7200)
            if "error" in res:
                raise RuntimeError(res["error"][0].data.decode(errors="replace"))
            lat.append(time.time() - t0)
            sizes.append(sum(len(c.data) for c in res[outs[0]]))
        out.update(value=round(statistics.median(lat), 3), latencies_s=[round(x, 3) for x in lat],
                   s_per_step=round(statistics.median(lat) / kw["num_steps"], 4), result_bytes=sizes,
                   higher_is_better=False)
    except Exception as e:  # noqa: BLE001
        out["error"] = f"{type(e).__name__}: {e}"
    finally:
        srv.shutdown()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=["bagel_t2i", "cosmos3_t2v"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--sp", type=int, default=1)
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--frames", type=int, default=93)
    ap.add_argument("--steps", type=int, default=None, help="override the number of denoise steps (reported)")
    ap.add_argument("--small", action="store_true", help="test-sized weights (CPU smoke run)")
    a = ap.parse_args()
    print(json.dumps(run_workload(a.workload, a.gpus, requests=a.requests, tp=a.tp, sp=a.sp, height=a.height,
                                  width=a.width, frames=a.frames, steps=a.steps, small=a.small)))


if __name__ == "__main__":
    main()
