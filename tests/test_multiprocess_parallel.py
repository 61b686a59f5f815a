"""Tensor- / sequence-parallel instances SERVED across OS processes on CPU (gloo): one process per rank, the ranks
of an instance in lockstep behind its first rank, single-rank nodes (encoders, codecs, autoencoders) beside them on
the same or on other ranks. Every placement must give what one rank gives.

What these cover in the worker / deployment: the process group spans only the ranks of parallel instances; a rank
trails its leader without booking the old walk's completion on the new walk; persisted tensors reach the followers;
only the first rank talks to the client, the conductor and other workers about a sharded node; a follower schedules
and reports the single-rank nodes it hosts; outputs of a single-rank node reach every rank of the instance they
feed; empty tensors cross the shared-memory arena."""
import hashlib
import os

import pytest
import torch

from mstar_b200.api_server.server import APIServer
from mstar_b200.conductor.deployment import load_config

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


def _serve(cfg_or_name, in_process, request, timeout=120, keep_bytes=False):
    cfg = load_config(os.path.join(ROOT, cfg_or_name)) if isinstance(cfg_or_name, str) else dict(cfg_or_name)
    if cfg["model"] != "tiny":
        cfg["model_kwargs"] = dict(cfg.get("model_kwargs") or {}, small=True)
    cfg["use_cuda_graphs"] = False
    torch.manual_seed(0)
    s = APIServer(cfg, in_process=in_process).start(240)
    try:
        prompt, outs, kw, tensors = request
        r = s.collect_results(s.submit_request(prompt, output_modalities=outs, model_kwargs=kw, tensors=tensors), timeout)
        assert "error" not in r, r["error"][0].data
        if keep_bytes:
            return {m: b"".join(c.data for c in r[m]) for m in outs}
        return {m: (len(r[m]), sum(len(c.data) for c in r[m]), hashlib.md5(b"".join(c.data for c in r[m])).hexdigest())
                for m in outs}
    finally:
        s.shutdown()


@pytest.fixture(autouse=True)
def _cpu_only(monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")


def test_tiny_decoder_tp2_over_processes_gives_the_single_rank_tokens():
    base = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128}}
    req = ("1 2 3 4", ["text"], dict(max_tokens=6, temperature=0.0), None)
    one = _serve(dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0]}]), True, req)
    two = _serve(dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0, 1], "tp_size": 2}]), False, req)
    assert two == one and one["text"][0] == 6          # six chunks: the follower rank sends nothing to the client


def test_orpheus_tp2_with_the_codec_on_one_of_its_ranks():
    req = ("hello there", ["audio"], dict(max_tokens=70, ignore_eos=True, temperature=0.0), None)
    got, want = _serve("orpheus_tp2.yaml", False, req), _serve("orpheus.yaml", True, req)
    assert got["audio"][:2] == want["audio"][:2] and want["audio"][1] > 0      # the codec adds noise: sizes, not samples


def test_qwen3_omni_thinker_and_talker_tp2_with_encoders_and_codec_beside_them():
    gen = torch.Generator().manual_seed(1)
    tens = {"audio": [torch.randn(8000, generator=gen) * 0.1], "image": [torch.rand(3, 16, 16, generator=gen)]}
    req = ("describe", ["text", "audio"], dict(max_tokens=6, ignore_eos=True, temperature=0.0, max_audio_tokens=12), tens)
    want = _serve("qwen3_omni.yaml", True, req)
    got = _serve("qwen3_omni_full_tp2.yaml", False, req)        # four ranks: thinker 0-1, talker 2-3
    assert got["text"] == want["text"] and got["audio"][:2] == want["audio"][:2]


def test_cosmos3_tp2_x_sp2_served_video_equals_the_single_rank_video():
    req = ("a robot", ["video"], dict(height=32, width=32, num_frames=5, num_steps=3, guidance_scale=4.0, seed=1), None)
    want = _frames(_serve("cosmos3_nano.yaml", True, req, keep_bytes=True)["video"])
    got = _frames(_serve("cosmos3_nano_tp2_sp2.yaml", False, req, keep_bytes=True)["video"])   # dit on four ranks
    assert got.shape == want.shape and got.shape[0] == 5
    # the sharded sums round differently in the last bit: a pixel that flips a grey level moves its JPEG block a little
    diff = abs(got.astype(int) - want.astype(int))
    assert diff.max() <= 6 and diff.mean() < 0.05 and want.std() > 10


def _frames(avi: bytes):
    """The JPEG frames of a Motion-JPEG AVI as one uint8 array [frames, H, W, 3]."""
    import io
    import numpy as np
    from PIL import Image
    out, pos = [], 0
    while True:
        a = avi.find(b"\xff\xd8", pos)
        if a < 0:
            break
        b = avi.find(b"\xff\xd9", a)
        out.append(np.asarray(Image.open(io.BytesIO(avi[a:b + 2])).convert("RGB")))
        pos = b + 2
    return np.stack(out)


def test_qwen3_omni_experts_cut_by_expert_over_four_ranks():
    """The layout of ``configs/qwen3_omni_ep8.yaml`` at test size: thinker and talker share ONE four-rank instance
    (attention tensor-parallel, every rank holding a quarter of the experts), encoders beside the first rank, the codec
    beside the last."""
    tens = {"audio": [torch.randn(8000, generator=torch.Generator().manual_seed(1)) * 0.1]}
    req = ("describe", ["text", "audio"], dict(max_tokens=6, ignore_eos=True, temperature=0.0, max_audio_tokens=12), tens)
    want = _serve("qwen3_omni.yaml", True, req)
    ep = {"model": "qwen3_omni", "model_kwargs": {"expert_parallel": True},
          "node_groups": [{"node_names": ["Thinker", "Talker"], "ranks": [0, 1, 2, 3], "tp_size": 4},
                          {"node_names": ["audio_encoder", "vision_encoder"], "ranks": [0]},
                          {"node_names": ["Code2Wav"], "ranks": [3]}]}
    got = _serve(ep, False, req)
    assert got["text"] == want["text"] and got["audio"][:2] == want["audio"][:2]


def test_wan22_dit_tp2_served_video_matches_the_single_rank_video():
    """``configs/wan22_tp2.yaml`` at test size: the AdaLN transformer on two ranks, text encoder beside the first,
    autoencoder beside the second."""
    req = ("a boat", ["video"], dict(height=32, width=32, num_frames=5, num_steps=3, guidance_scale=4.0, seed=1), None)
    want = _frames(_serve("wan22.yaml", True, req, keep_bytes=True)["video"])
    got = _frames(_serve("wan22_tp2.yaml", False, req, keep_bytes=True)["video"])
    assert got.shape == want.shape
    diff = abs(got.astype(int) - want.astype(int))
    assert diff.max() <= 6 and diff.mean() < 0.05 and want.std() > 10


def test_wan22_dit_tp2_x_sp2_served_video_matches_the_single_rank_video():
    req = ("a boat", ["video"], dict(height=32, width=32, num_frames=5, num_steps=3, guidance_scale=4.0, seed=1), None)
    want = _frames(_serve("wan22.yaml", True, req, keep_bytes=True)["video"])
    got = _frames(_serve("wan22_tp2_sp2.yaml", False, req, keep_bytes=True)["video"])
    assert got.shape == want.shape
    diff = abs(got.astype(int) - want.astype(int))
    assert diff.max() <= 6 and diff.mean() < 0.05 and want.std() > 10
