"""OpenAI-compatible media routes in front of the model families (test-sized weights, CPU): speech, images
(generation and edit with an uploaded file), videos."""
import base64
import io

import pytest
import torch
from fastapi.testclient import TestClient

from mstar_b200.api_server.app import create_app
from mstar_b200.api_server.media_io import tensor_to_png
from mstar_b200.api_server.server import APIServer


def _client(cfg):
    s = APIServer(cfg, in_process=True).start(120)
    return s, TestClient(create_app(s))


def test_speech_route_orpheus():
    s, c = _client({"model": "orpheus", "model_kwargs": {"small": True, "page_size": 16, "max_num_pages": 256},
                    "use_cuda_graphs": False,
                    "node_groups": [{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                                    {"node_names": ["snac_decoder"], "ranks": [1], "graph_walks": ["snac_chunk"]}]})
    try:
        r = c.post("/v1/audio/speech", json={"model": "orpheus", "input": "hello", "voice": "leo", "response_format": "wav",
                                             "max_tokens": 35, "ignore_eos": True})
        assert r.status_code == 200 and r.content[:4] == b"RIFF" and len(r.content) > 44 + 2048 * 2
        r = c.post("/v1/audio/speech", json={"model": "orpheus", "input": "hello", "response_format": "pcm", "stream": True,
                                             "max_tokens": 35, "ignore_eos": True})
        assert r.status_code == 200 and len(r.content) >= 2048 * 2
    finally:
        s.shutdown()


def test_image_routes_bagel():
    s, c = _client({"model": "bagel", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
                    "node_groups": [{"node_names": ["vit_encoder", "vae_encoder", "LLM", "vae_decoder", "LLM_cfg_text",
                                                    "LLM_cfg_img", "combine_cfg"], "ranks": [0]}]})
    try:
        r = c.post("/v1/images/generations", json={"model": "bagel", "prompt": "a cat", "n": 2, "size": "16x16", "seed": 3,
                                                   "num_steps": 2})
        assert r.status_code == 200, r.text
        imgs = [base64.b64decode(d["b64_json"]) for d in r.json()["data"]]
        assert len(imgs) == 2 and all(i[:4] == b"\x89PNG" for i in imgs) and imgs[0] != imgs[1]
        png = tensor_to_png(torch.rand(3, 16, 16))
        r = c.post("/v1/images/edits", data={"prompt": "make it blue", "size": "16x16", "seed": "1"},
                   files={"image": ("in.png", io.BytesIO(png), "image/png")})
        assert r.status_code == 200, r.text
        assert base64.b64decode(r.json()["data"][0]["b64_json"])[:4] == b"\x89PNG"
    finally:
        s.shutdown()


def test_video_route_wan22():
    s, c = _client({"model": "wan22", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
                    "node_groups": [{"node_names": ["text_encoder", "vae_encoder", "dit", "vae_decoder"], "ranks": [0]}]})
    try:
        r = c.post("/v1/videos/generations", json={"model": "wan22", "prompt": "waves", "size": "16x16", "num_frames": 5,
                                                   "seed": 1, "num_steps": 2})
        assert r.status_code == 200, r.text
        assert base64.b64decode(r.json()["data"][0]["b64_json"])[:4] == b"RIFF"
    finally:
        s.shutdown()
