"""The benchmark client against a served tiny model (uvicorn on CPU) and its metric arithmetic."""
import asyncio
import socket
import threading
import time

from mstar_b200.benchmark.metrics import RequestMetrics, aggregate
from mstar_b200.benchmark.requests import make_requests, synthetic_png, synthetic_wav
from mstar_b200.benchmark.runner import BenchmarkRunner


def test_metric_arithmetic():
    m = RequestMetrics("r", "tts", t_send=10.0)
    for k in range(4):                      # 4 chunks of 0.1 s audio arriving every 0.05 s, then one late chunk
        m.record("audio", 4800, 10.2 + 0.05 * k)
    m.record("audio", 4800, 10.2 + 0.15 + 0.3)
    m.t_done = 11.0
    assert abs(m.ttft["audio"] - 0.2) < 1e-9 and abs(m.audio_seconds() - 0.5) < 1e-9
    assert m.streaming_viability() == 0.75          # the last gap (0.3 s) exceeded the 0.1 s the previous chunk held
    t = RequestMetrics("t", "t2t", t_send=0.0)
    t.record("text", 10, 0.1, units=2)
    t.record("text", 10, 0.3, units=2)
    t.t_done = 0.3
    assert abs(t.itl("text")[0] - 0.1) < 1e-9       # 0.2 s between chunks of two tokens each
    agg = aggregate([m, t], wall_s=2.0, mode="offline")
    assert agg.n_success == 2 and agg.text_tokens_per_s == 2.0 and abs(agg.audio_seconds_per_s - 0.25) < 1e-9
    assert abs(agg.rtf.p50 - 2.0) < 1e-9 and "TTFT (audio" in str(agg)


def test_synthetic_inputs_are_valid_files():
    import random
    import wave
    import io
    png = synthetic_png(8, 8, random.Random(0))
    assert png[:8] == b"\x89PNG\r\n\x1a\n"
    with wave.open(io.BytesIO(synthetic_wav(0.1, random.Random(0))), "rb") as w:
        assert w.getframerate() == 16000 and w.getnframes() == 1600
    assert make_requests("i2t", 2, image_size=8)[0].files[0][0].endswith(".png")


def test_closed_loop_run_against_a_served_tiny_model():
    import uvicorn
    from mstar_b200.api_server.app import create_app
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128},
           "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
    srv = APIServer(cfg, in_process=True).start(60)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    us = uvicorn.Server(uvicorn.Config(create_app(srv), host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=us.run, daemon=True)
    th.start()
    try:
        for _ in range(100):
            if us.started:
                break
            time.sleep(0.05)
        reqs = make_requests("t2t", 6, max_tokens=5, numeric_prompts=True, extra_kwargs={"temperature": 0.0})
        ms, agg = asyncio.run(BenchmarkRunner(f"http://127.0.0.1:{port}", reqs, mode="closed_loop", max_concurrency=3,
                                              warmup=1).run())
        assert agg.n_success == 6, agg.errors
        assert all(m.units["text"] == 5 for m in ms)
        assert agg.ttft["text"].p50 > 0 and agg.text_tokens_per_s > 0 and agg.e2e.p99 >= agg.e2e.p50
    finally:
        us.should_exit = True
        th.join(5)
        srv.shutdown()
