"""End-to-end serving benchmark of the TTS deployment through the public server, the way a user runs it: ONE
deployment with a conductor process and one worker process per GPU (every GPU holds an LLM replica and a codec
replica, placed by the same YAML keys a config file uses), the C++ HTTP frontend in front, and 64 concurrent
streaming requests per GPU over ``POST /generate``. Tokens are counted from the audio that the clients receive
(7 tokens per 2048 samples of 16-bit audio) inside the window in which all requests decode; time to first audio is
taken under that same load. ``baseline/reference_bench.py`` measures the reference the same way with the same
client, so the two numbers compare like for like.

    python -m mstar_b200.bench.serve_tts --gpus 1 --concurrency 64 --tokens 1204 [--small] [--uvicorn] [--in-process]
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import socket
import tempfile
import threading
import time

from .tts_client import run_streams, summarize


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def deployment_config(n_gpus: int, concurrency: int, *, small: bool = False, codec_dtype: str = "float32",
                      tp: int = 1, max_num_pages: int = 2048) -> dict:
    """LLM replicas on every rank (or one tensor-parallel instance per ``tp`` ranks) and a codec replica on every
    rank: repeated ranks of a node group without ``tp_size`` are data-parallel replicas."""
    ranks = list(range(n_gpus))
    llm = {"node_names": ["LLM"], "ranks": ranks, "graph_walks": ["prefill", "decode"]}
    if tp > 1:
        llm["tp_size"] = tp
    return {"model": "orpheus",
            "model_kwargs": {"small": small, "page_size": 16 if small else 128, "max_num_pages": max_num_pages,
                             "codec_dtype": codec_dtype},
            "max_batch_size": max(64, concurrency),
            "max_concurrent_requests": max(256, 2 * concurrency * n_gpus),
            "node_groups": [llm, {"node_names": ["snac_decoder"], "ranks": ranks, "graph_walks": ["snac_chunk"]}]}


def run_serving(n_gpus: int = 1, concurrency: int = 64, tokens: int = 1204, *, small: bool = False,
                uvicorn_frontend: bool = False, in_process: bool = False, codec_dtype: str = "float32", tp: int = 1,
                warm_tokens: int = 56, trace_out: str | None = None) -> dict:
    """Start the deployment, warm it up (one request, then a short round at full concurrency that captures every
    batch bucket), run the measured round and shut down. Returns the summary with the workers' own counters."""
    from ..api_server.app import create_app
    from ..api_server.server import APIServer
    total = concurrency * max(1, n_gpus // tp)
    stats_dir = tempfile.mkdtemp(prefix="mstar_stats_")
    os.environ["MSTAR_WORKER_STATS_DIR"] = stats_dir
    if trace_out:
        os.environ["MSTAR_TRACE_WORKER"] = "1"
    cfg = deployment_config(n_gpus, concurrency, small=small, codec_dtype=codec_dtype, tp=tp)
    out = {"bench": "serve_tts", "n_gpus": n_gpus, "concurrency": total, "tokens_per_request": tokens,
           "frontend": "uvicorn" if uvicorn_frontend else "mstar-server", "multi_process": not in_process,
           "codec_dtype": codec_dtype, "tp": tp}
    srv = APIServer(cfg, in_process=in_process).start(1800)
    port = _free_port()
    app = create_app(srv)
    fe = None
    try:
        if uvicorn_frontend:
            import uvicorn
            us = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
            threading.Thread(target=us.run, daemon=True).start()
        else:
            from ..api_server.native_frontend import NativeFrontend
            fe = NativeFrontend(app, "127.0.0.1", port).start()
        url = f"http://127.0.0.1:{port}/generate"
        import requests
        for _ in range(400):
            try:
                if requests.get(f"http://127.0.0.1:{port}/health", timeout=1).status_code == 200:
                    break
            except Exception:  # noqa: BLE001
                time.sleep(0.05)
        kw = {"ignore_eos": True, "voice": "tara"}
        w = run_streams(url, 1, dict(kw, max_tokens=28 * 3), text="warm up")
        if w[0]["error"] or not w[0]["chunks"]:
            raise RuntimeError(f"warm-up failed: {w[0]['error'] or 'no audio'}")
        run_streams(url, total, dict(kw, max_tokens=warm_tokens), text="warm {i}")
        recs = run_streams(url, total, dict(kw, max_tokens=tokens))
        if trace_out:
            out["client"] = [{"t_submit": r["t_submit"], "t_first": r["t_first"], "t_done": r["t_done"],
                              "n_chunks": len(r["chunks"])} for r in recs]
        s = summarize(recs, total)
        out.update(tokens_per_s=round(s["tokens_per_s"], 1), window_s=round(s["window_s"], 3),
                   ttfa_p50_ms=round(s["ttfa_p50_ms"], 1), ttfa_p99_ms=round(s["ttfa_p99_ms"], 1),
                   ms_per_step=round(1e3 * concurrency * max(1, n_gpus // tp) / max(s["tokens_per_s"], 1e-9), 3),
                   audio_tokens_total=round(s["audio_tokens_total"]), wall_s=round(s["wall_s"], 3))
    except Exception as e:  # noqa: BLE001
        out["error"] = f"{type(e).__name__}: {e}"
    finally:
        if fe is not None:
            fe.stop()
        if in_process:
            out["workers"] = [w_.stats() for w_ in srv.deployment.workers]
        srv.shutdown()
        os.environ.pop("MSTAR_WORKER_STATS_DIR", None)
    if not in_process:
        out["workers"] = []
        for f in sorted(glob.glob(os.path.join(stats_dir, "*.json"))):
            try:
                with open(f) as fh:
                    out["workers"].append(json.load(fh))
            except Exception:  # noqa: BLE001
                pass
    shutil.rmtree(stats_dir, ignore_errors=True)
    if trace_out:
        os.environ.pop("MSTAR_TRACE_WORKER", None)
        with open(trace_out, "w") as f:
            json.dump(out, f)
        for w_ in out.get("workers", []):
            w_.pop("trace", None)
        out.pop("client", None)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--concurrency", type=int, default=64, help="concurrent requests per model replica")
    ap.add_argument("--tokens", type=int, default=1204)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--small", action="store_true", help="test-sized weights (CPU smoke run)")
    ap.add_argument("--uvicorn", action="store_true", help="FastAPI / uvicorn frontend instead of mstar-server")
    ap.add_argument("--in-process", action="store_true", help="conductor and workers as threads of this process")
    ap.add_argument("--codec-dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--trace-out", default=None, help="write the workers' batch timeline and the clients' times here")
    a = ap.parse_args()
    print(json.dumps(run_serving(a.gpus, a.concurrency, a.tokens, small=a.small, uvicorn_frontend=a.uvicorn,
                                 in_process=a.in_process, codec_dtype=a.codec_dtype, tp=a.tp,
                                 trace_out=a.trace_out)))


if __name__ == "__main__":
    main()
