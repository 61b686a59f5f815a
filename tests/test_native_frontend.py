"""The C++ HTTP frontend (`mstar-server`) in front of the in-process deployment: same routes and payloads as the
uvicorn frontend, chunked streaming, concurrent connections, native health / stats."""
import base64
import json
import os
import socket
import threading
import time

import pytest
import requests

from mstar_b200.api_server.app import create_app
from mstar_b200.api_server.native_frontend import LIB_DIR, NativeFrontend
from mstar_b200.api_server.server import APIServer

pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(LIB_DIR, "mstar-server")),
                                reason="native frontend binary not built")

CFG = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128},
       "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def base_url():
    srv = APIServer(CFG, in_process=True).start(60)
    port = _free_port()
    fe = NativeFrontend(create_app(srv), "127.0.0.1", port).start()
    url = f"http://127.0.0.1:{port}"
    for _ in range(100):
        try:
            if requests.get(url + "/health", timeout=1).status_code == 200:
                break
        except Exception:  # noqa: BLE001
            pass
        time.sleep(0.05)
    yield url
    fe.stop()
    srv.shutdown()


def test_health_models_and_native_stats(base_url):
    assert requests.get(base_url + "/health", timeout=5).json() == {"status": "healthy"}
    assert requests.get(base_url + "/v1/models", timeout=5).json()["data"][0]["id"] == "tiny"
    st = requests.get(base_url + "/frontend_stats", timeout=5).json()
    assert st["served"] >= 2 and st["errors"] == 0
    assert requests.get(base_url + "/nope", timeout=5).status_code == 404


def test_generate_plain_and_chunked_stream(base_url):
    kw = json.dumps({"max_tokens": 5, "temperature": 0.0})
    r = requests.post(base_url + "/generate", data={"text": "1 2 3", "streaming": "false", "model_kwargs": kw}, timeout=60)
    assert r.status_code == 200 and "content-length" in {k.lower() for k in r.headers}
    toks = b"".join(base64.b64decode(c["data"]) for c in r.json()["outputs"]["text"]).decode().split()
    assert len(toks) == 5
    with requests.post(base_url + "/generate", data={"text": "1 2 3", "streaming": "true", "model_kwargs": kw},
                       stream=True, timeout=60) as r:
        assert r.headers.get("Transfer-Encoding") == "chunked"
        lines = [json.loads(l) for l in r.iter_lines() if l]
    assert "".join(base64.b64decode(l["data"]).decode() for l in lines).split() == toks
    bad = requests.post(base_url + "/generate", data={"text": "x", "model_kwargs": "{nope"}, timeout=10)
    assert bad.status_code == 400


def test_openai_chat_sse_through_native_frontend(base_url):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "1 2 3"}], "max_tokens": 3, "temperature": 0,
            "stream": True}
    with requests.post(base_url + "/v1/chat/completions", json=body, stream=True, timeout=60) as r:
        events = [l[6:].decode() for l in r.iter_lines() if l.startswith(b"data: ")]
    assert events[-1] == "[DONE]" and len(events) >= 4


def test_many_concurrent_connections(base_url):
    kw = json.dumps({"max_tokens": 3, "temperature": 0.0})
    out, errs = [], []

    def one(i):
        try:
            r = requests.post(base_url + "/generate", data={"text": f"{i} 2 3", "streaming": "false", "model_kwargs": kw},
                              timeout=120)
            out.append(r.status_code)
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))
    ts = [threading.Thread(target=one, args=(i,)) for i in range(24)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs and out.count(200) == 24
