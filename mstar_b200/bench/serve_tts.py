"""End-to-end serving benchmark of the TTS placement through the public server: N concurrent streaming requests
over HTTP (C++ frontend or uvicorn), LLM and codec partitions on one GPU, tokens counted from the audio received
(7 tokens per 2048 samples of 16-bit audio) inside the window in which all requests decode. The same measurement as
the reference arm of bench.py (baseline/reference_bench.py), so the two numbers compare like for like.

    python -m mstar_b200.bench.serve_tts --concurrency 64 --tokens 1204 [--small] [--uvicorn]
"""
from __future__ import annotations

import argparse
import json
import socket
import statistics
import threading
import time


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Stream(threading.Thread):
    def __init__(self, url, text, max_tokens):
        super().__init__(daemon=True)
        self.url, self.text, self.max_tokens = url, text, max_tokens
        self.t_submit = self.t_first = self.t_done = None
        self.chunks, self.error = [], None

    def run(self):
        import base64

        import requests
        try:
            self.t_submit = time.perf_counter()
            data = {"text": self.text, "output_modalities": "audio", "streaming": "true",
                    "model_kwargs": json.dumps({"max_tokens": self.max_tokens, "ignore_eos": True, "voice": "tara"})}
            with requests.post(self.url, data=data, stream=True, timeout=1800) as r:
                r.raise_for_status()
                for line in r.iter_lines():
                    if not line:
                        continue
                    msg = json.loads(line)
                    if msg.get("modality") == "error":
                        self.error = base64.b64decode(msg.get("data", "")).decode(errors="replace")
                        break
                    n = len(base64.b64decode(msg.get("data") or ""))
                    if msg.get("modality") == "audio" and n:
                        now = time.perf_counter()
                        self.t_first = self.t_first or now
                        self.chunks.append((now, n))
        except Exception as e:  # noqa: BLE001
            self.error = f"{type(e).__name__}: {e}"
        self.t_done = time.perf_counter()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=1204)
    ap.add_argument("--small", action="store_true", help="test-sized weights (CPU smoke run)")
    ap.add_argument("--uvicorn", action="store_true", help="FastAPI / uvicorn frontend instead of mstar-server")
    ap.add_argument("--multi-process", action="store_true")
    ap.add_argument("--codec-dtype", default="float32", choices=["float32", "bfloat16"])
    a = ap.parse_args()
    from ..api_server.app import create_app
    from ..api_server.server import APIServer
    cfg = {"model": "orpheus",
           "model_kwargs": {"small": a.small, "page_size": 16 if a.small else 128,
                            "max_num_pages": 2048, "codec_dtype": a.codec_dtype},
           "max_batch_size": max(64, a.concurrency),
           "node_groups": [{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                           {"node_names": ["snac_decoder"], "ranks": [0], "graph_walks": ["snac_chunk"]}]}
    srv = APIServer(cfg, in_process=not a.multi_process).start(900)
    port = _free_port()
    app = create_app(srv)
    fe = None
    if a.uvicorn:
        import uvicorn
        config = uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning")
        us = uvicorn.Server(config)
        threading.Thread(target=us.run, daemon=True).start()
    else:
        from ..api_server.native_frontend import NativeFrontend
        fe = NativeFrontend(app, "127.0.0.1", port).start()
    url = f"http://127.0.0.1:{port}/generate"
    import requests
    for _ in range(200):
        try:
            if requests.get(f"http://127.0.0.1:{port}/health", timeout=1).status_code == 200:
                break
        except Exception:  # noqa: BLE001
            time.sleep(0.05)
    out = {"bench": "serve_tts", "concurrency": a.concurrency, "tokens_per_request": a.tokens,
           "frontend": "uvicorn" if a.uvicorn else "mstar-server", "multi_process": a.multi_process,
           "codec_dtype": a.codec_dtype}
    try:
        w = _Stream(url, "warm up", 28 * 3)
        w.start()
        w.join(900)
        if w.error or not w.chunks:
            raise RuntimeError(f"warm-up failed: {w.error or 'no audio'}")
        # second warm-up at full concurrency for a few frames: captures the decode graphs of every batch bucket
        ws = [_Stream(url, f"warm {i}", 28 * 2) for i in range(a.concurrency)]
        for s in ws:
            s.start()
        for s in ws:
            s.join(900)
        streams = [_Stream(url, f"request number {i} says hello", a.tokens) for i in range(a.concurrency)]
        for s in streams:
            s.start()
        for s in streams:
            s.join(1800)
        bad = [s.error for s in streams if s.error or not s.chunks]
        if bad:
            raise RuntimeError(f"{len(bad)} of {a.concurrency} requests failed: {bad[0]}")
        t_open, t_close = max(s.t_first for s in streams), min(s.t_done for s in streams)
        nbytes = sum(b for s in streams for (t, b) in s.chunks if t_open < t <= t_close)
        tokens = nbytes / 2 / 2048 * 7
        dt = t_close - t_open
        out.update(tokens_per_s=round(tokens / dt, 1), window_s=round(dt, 3),
                   ttfa_p50_ms=round(statistics.median((s.t_first - s.t_submit) * 1e3 for s in streams), 1),
                   ms_per_step=round(1e3 * a.concurrency * dt / max(tokens, 1), 3))
    except Exception as e:  # noqa: BLE001
        out["error"] = f"{type(e).__name__}: {e}"
    finally:
        if fe is not None:
            fe.stop()
        srv.shutdown()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
