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


def test_frontend_encodes_batched_binary_chunks_like_python():
    """Chunks stated as prefix + base64(data) + suffix are collected, sent to the frontend as ONE frame and encoded
    there: every padding case, binary bytes, chunks of several requests in one batch, and frame order (head, batched
    chunks, a plain piece, end) survive."""
    datas = [bytes(range(n)) for n in range(8)] + [os.urandom(5461), os.urandom(4096)]
    fe_box = {}

    async def app(scope, receive, send):
        await receive()
        direct = scope["extensions"]["mstar.direct_stream"]
        await send({"type": "http.response.start", "status": 200, "headers": [(b"content-type", b"text/plain")]})
        for d in datas:
            direct.b64(b"<", d, b">\n")
        fe_box["fe"]._flush_batch()         # what the API server's after-message hook does
        direct.b64(b"<", b"late", b">\n")
        direct(b"plain\n")                  # a plain piece flushes what was collected before it
        await send({"type": "http.response.body", "body": b"", "more_body": False})

    class _State:
        pass

    class _Srv:
        after_message_hooks: list = []
    app.state = _State()
    app.state.mstar_server = _Srv()
    port = _free_port()
    fe = fe_box["fe"] = NativeFrontend(app, "127.0.0.1", port).start()
    try:
        assert fe._batching and _Srv.after_message_hooks == [fe._flush_batch]
        bodies = []

        def get():
            bodies.append(requests.get(f"http://127.0.0.1:{port}/x", timeout=20).content)
        ts = [threading.Thread(target=get) for _ in range(3)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        want = b"".join(b"<" + base64.b64encode(d) + b">\n" for d in datas + [b"late"]) + b"plain\n"
        assert bodies == [want] * 3
        assert fe.stats["batched_chunks"] == 3 * (len(datas) + 1) and fe.stats["batches"] >= 3
    finally:
        fe.stop()


def test_plain_form_parser_accepts_text_fields_only():
    from mstar_b200.api_server.app import _simple_form
    assert _simple_form(b"text=1+2+3&streaming=true&model_kwargs=%7B%22max_tokens%22%3A+5%7D",
                        "application/x-www-form-urlencoded") == {"text": "1 2 3", "streaming": "true",
                                                                 "model_kwargs": '{"max_tokens": 5}'}
    assert _simple_form(b"text=a&text=b", "application/x-www-form-urlencoded") is None            # repeated field
    assert _simple_form(b"text=a&surprise=1", "application/x-www-form-urlencoded") is None        # unknown field
    b = "XyZ"
    body = (f'--{b}\r\nContent-Disposition: form-data; name="text"\r\n\r\nhello\r\nworld\r\n'
            f'--{b}\r\nContent-Disposition: form-data; name="streaming"\r\n\r\ntrue\r\n--{b}--\r\n').encode()
    assert _simple_form(body, f"multipart/form-data; boundary={b}") == {"text": "hello\r\nworld", "streaming": "true"}
    upload = (f'--{b}\r\nContent-Disposition: form-data; name="files"; filename="a.wav"\r\n'
              f'Content-Type: audio/wav\r\n\r\nRIFF\r\n--{b}--\r\n').encode()
    assert _simple_form(upload, f"multipart/form-data; boundary={b}") is None                      # a file part
    assert _simple_form(body[:-8], f"multipart/form-data; boundary={b}") is None                   # no closing delimiter
    assert _simple_form(b"{}", "application/json") is None


def test_streaming_generate_takes_the_framework_free_route_and_equals_the_full_route(base_url):
    """Form posts without uploads (urlencoded or multipart) are served without the web framework's parsing and routing
    layers under the C++ frontend and give the same stream; malformed input still gets the full route's error."""
    kw = json.dumps({"max_tokens": 5, "temperature": 0.0})
    before = requests.get(base_url + "/frontend_stats", timeout=5).json()

    def stream(extra):
        with requests.post(base_url + "/generate", data=dict({"text": "4 5 6", "streaming": "true", "model_kwargs": kw}, **extra),
                           stream=True, timeout=60) as r:
            assert r.status_code == 200
            return [json.loads(l) for l in r.iter_lines() if l]
    fast = stream({})
    multipart = requests.post(base_url + "/generate", files={"text": (None, "4 5 6"), "streaming": (None, "true"),
                                                             "model_kwargs": (None, kw)}, stream=True, timeout=60)
    slow = [json.loads(l) for l in multipart.iter_lines() if l]
    assert [l["data"] for l in fast] == [l["data"] for l in slow] and len(fast) == 5
    bad = requests.post(base_url + "/generate", data={"text": "x", "model_kwargs": "{nope"}, timeout=10)
    assert bad.status_code == 400                       # malformed input still gets the full route's error
    assert before is not None
