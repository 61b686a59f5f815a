"""Capacity of the API process alone: how many streamed audio chunks per second it can take from workers and hand to
HTTP clients, and how long it needs to take in a burst of simultaneous requests.

Nothing here runs a model. A stand-in for the workers (a thread with its own mailbox and tensor store) emits one
2048-sample PCM chunk per active request and frame period, as batches of result messages like a worker's; the real
API server, the real C++ frontend (or uvicorn) and real client processes do the rest. With ``--frame-s 0`` the
producer emits as fast as it is acknowledged (capacity); with the serving frame period (0.03) it shows the intake of
a burst and the chunk rate a deployment of that many streams needs.

    python -m mstar_b200.bench.api_capacity --streams 256 --frames 100 [--frame-s 0.03]

The producer shares the interpreter with the API server here, so the numbers are a lower bound of what the API
process does when the workers are other processes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time


def run(streams: int = 256, frames: int = 100, frame_s: float = 0.0) -> dict:
    import torch

    from ..api_server.app import create_app
    from ..api_server.native_frontend import NativeFrontend
    from ..api_server.server import APIServer
    from ..communication.communicator import LocalCommunicator
    from ..communication.tensors import TensorCommunicationManager
    from ..utils import ipc_format as ipc
    from ..utils.ipc_format import Message
    from .serve_tts import _free_port, deployment_config
    from .tts_client import run_streams

    sys.setswitchinterval(0.005)
    srv = APIServer(deployment_config(1, streams, small=True), in_process=True)
    dep = srv.deployment
    cond = LocalCommunicator("conductor", dep.hub)
    wcomm = LocalCommunicator("worker_0", dep.hub)
    tens = TensorCommunicationManager("worker_0", torch.device("cpu"), arena_prefix=dep.prefix)
    state = {"stop": False}
    seen: list[float] = []

    def producer():
        active: dict[str, int] = {}
        audio = (torch.randn(2048) * 3000).to(torch.int16)
        while not state["stop"]:
            for m in cond.recv_or_wake(0.0005 if active else 0.05):
                if m.type == ipc.ConductorMessageType.NEW_REQUEST:
                    active[m.body.request_id] = 0
                    seen.append(time.time())
            for _ in wcomm.recv_or_wake(0.0):
                pass
            items = []
            for rid in list(active):
                ti = tens.prepare_for_remote(tens.store_and_return_tensor_info(rid + "#emit", audio.clone()), "api")
                items.append(ipc.ResultTensors(rid, "audio", [ti], {"name": "audio"}, "worker_0"))
            if items:
                wcomm.send("api", Message(ipc.ApiMessageType.RESULT_TENSORS_BATCH, ipc.ResultTensorsBatch(items)))
            for rid in list(active):
                active[rid] += 1
                if active[rid] >= frames:
                    del active[rid]
                    cond.send("api", Message(ipc.ApiMessageType.REQUEST_COMPLETE, ipc.RequestComplete(rid, {})))
            if active and frame_s:
                time.sleep(frame_s)

    busy = {"s": 0.0, "n": 0}
    handle = srv._handle

    def timed(m):
        t = time.perf_counter()
        handle(m)
        busy["s"] += time.perf_counter() - t
        busy["n"] += len(getattr(m.body, "items", ())) or 1
    srv._handle = timed
    dep.threads = [threading.Thread(target=producer, daemon=True)]
    srv.ready.set()
    srv.start(10)
    port = _free_port()
    fe = NativeFrontend(create_app(srv), "127.0.0.1", port).start()
    try:
        time.sleep(0.5)
        t0 = time.time()
        recs = run_streams(f"http://127.0.0.1:{port}/generate", streams,
                           {"max_tokens": 7 * frames, "ignore_eos": True, "voice": "tara"})
        wall = time.time() - t0
        n = sum(len(r["chunks"]) for r in recs)
        t_open, t_close = max(r["t_first"] for r in recs), min(r["t_done"] for r in recs)
        inwin = sum(1 for r in recs for (t, _) in r["chunks"] if t_open < t <= t_close)
        return {"bench": "api_capacity", "streams": streams, "frames": frames, "frame_s": frame_s, "chunks": n,
                "chunks_per_s_all_streams_active": round(inwin / max(1e-9, t_close - t_open)),
                "result_thread_us_per_chunk": round(busy["s"] / max(1, busy["n"]) * 1e6, 1),
                "intake_ms_first_to_last_request": round((seen[-1] - seen[0]) * 1e3, 1) if seen else None,
                "frontend": dict(fe.stats), "wall_s": round(wall, 2),
                "errors": [r["error"] for r in recs if r["error"]][:2]}
    finally:
        state["stop"] = True
        fe.stop()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--streams", type=int, default=256)
    ap.add_argument("--frames", type=int, default=100)
    ap.add_argument("--frame-s", type=float, default=0.0)
    a = ap.parse_args()
    print(json.dumps(run(a.streams, a.frames, a.frame_s)))
    os._exit(0)          # client and frontend helper threads need no orderly shutdown here


if __name__ == "__main__":
    main()
