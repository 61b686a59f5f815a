"""HTTP surface over the in-process deployment: /generate (NDJSON + JSON), /health, /metrics, OpenAI routes,
and the Python SDK against a real uvicorn server."""
import base64
import json
import socket
import threading
import time

import pytest
from fastapi.testclient import TestClient

from mstar_b200.api_server.app import create_app
from mstar_b200.api_server.server import APIServer
from mstar_b200.client import MStarClient

CFG = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128},
       "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}


@pytest.fixture(scope="module")
def server():
    s = APIServer(CFG, in_process=True).start(60)
    yield s
    s.shutdown()


@pytest.fixture(scope="module")
def client(server):
    return TestClient(create_app(server))


def test_health_metrics_models(client):
    assert client.get("/health").json() == {"status": "healthy"}
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    m = client.get("/metrics").text
    assert "mstar_kv_pages_total" in m and "mstar_api_requests_submitted_total" in m


def test_generate_json_and_ndjson(client):
    kw = json.dumps({"max_tokens": 4, "temperature": 0.0})
    r = client.post("/generate", data={"text": "1 2 3", "streaming": "false", "model_kwargs": kw, "request_id": "abc"})
    assert r.status_code == 200
    doc = r.json()
    assert doc["request_id"] == "abc"
    toks = b"".join(base64.b64decode(c["data"]) for c in doc["outputs"]["text"]).decode().split()
    assert len(toks) == 4
    r = client.post("/generate", data={"text": "1 2 3", "streaming": "true", "model_kwargs": kw})
    lines = [json.loads(l) for l in r.text.strip().split("\n")]
    assert len(lines) == 4 and all(l["modality"] == "text" for l in lines)
    streamed = "".join(base64.b64decode(l["data"]).decode() for l in lines).split()
    assert streamed == toks                      # greedy: same prompt, same tokens
    assert client.post("/generate", data={"text": "x", "output_modalities": "smell"}).status_code == 400
    assert client.post("/generate", data={"text": "x", "model_kwargs": "{nope"}).status_code == 400


def test_openai_chat_stream_and_plain(client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "1 2 3"}], "max_tokens": 3, "temperature": 0}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200
    msg = r.json()["choices"][0]["message"]
    assert msg["role"] == "assistant" and len(msg["content"].split()) == 3
    r = client.post("/v1/chat/completions", json=dict(body, stream=True, top_k=5))   # extra field passes through
    events = [l[6:] for l in r.text.split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    deltas = [json.loads(e)["choices"][0]["delta"] for e in events[:-1]]
    assert deltas[0]["role"] == "assistant" and sum("content" in d for d in deltas) == 3
    r = client.post("/v1/chat/completions", json={"messages": "nope"})
    assert r.status_code == 422


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_python_sdk_against_uvicorn(server):
    import uvicorn
    port = _free_port()
    cfg = uvicorn.Config(create_app(server), host="127.0.0.1", port=port, log_level="warning")
    uv = uvicorn.Server(cfg)
    t = threading.Thread(target=uv.run, daemon=True)
    t.start()
    c = MStarClient(f"http://127.0.0.1:{port}", timeout=60)
    for _ in range(100):
        try:
            if c.health()["status"] == "healthy":
                break
        except Exception:
            time.sleep(0.1)
    res = c.generate("4 5 6", max_tokens=3, temperature=0.0)
    assert len(res.text.split()) == 3
    chunks = list(c.stream("4 5 6", max_tokens=3, temperature=0.0))
    assert "".join(ch.text for ch in chunks).split() == res.text.split()
    assert c.chat("4 5 6", max_tokens=2, temperature=0.0)
    uv.should_exit = True
    t.join(10)
