"""Every model family through the in-process serving stack on one GPU (all workers share cuda:0), test-sized bf16
weights whose shapes run on the tensor-core kernels, CUDA graphs on for the decode loops."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _server(cfg):
    from mstar_b200.api_server.server import APIServer
    return APIServer(cfg, in_process=True).start(300)


def _run(s, text, outs, timeout=300, tensors=None, **mk):
    res = s.collect_results(s.submit_request(text, output_modalities=outs, model_kwargs=mk, tensors=tensors), timeout)
    assert "error" not in res, res
    return res


def test_orpheus_tts_with_decode_graphs():
    s = _server({"model": "orpheus", "model_kwargs": {"small": True, "page_size": 128, "max_num_pages": 64},
                 "node_groups": [{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                                 {"node_names": ["snac_decoder"], "ranks": [1], "graph_walks": ["snac_chunk"]}]})
    try:
        res = _run(s, "hello there", ["audio"], max_tokens=63, ignore_eos=True)
        assert sum(len(c.data) for c in res["audio"]) >= 2048 * 2 * 6
        eng = s.deployment.workers[0].engines.engine_for("LLM")
        assert eng.graph_hits >= 50
        eng.check_status()
    finally:
        s.shutdown()


def test_wan22_video_and_cosmos3_walks():
    s = _server({"model": "wan22", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["text_encoder", "vae_encoder", "dit", "vae_decoder"], "ranks": [0]}]})
    try:
        kw = dict(num_steps=3, height=32, width=32, num_frames=5, seed=7)
        a = _run(s, "a red fox", ["video"], **kw)
        assert a["video"][0].data[:4] == b"RIFF"
        b = _run(s, "a red fox", ["video"], tensors={"image": [torch.rand(3, 32, 32) * 2 - 1]}, **kw)
        assert b["video"][0].data != a["video"][0].data
    finally:
        s.shutdown()
    s = _server({"model": "cosmos3", "model_kwargs": {"small": True, "page_size": 128, "max_num_pages": 32},
                 "node_groups": [{"node_names": ["dit", "vae_encoder", "vae_decoder", "audio_decoder"], "ranks": [0]}]})
    try:
        kw = dict(num_steps=3, height=32, width=32, num_frames=5, negative_prompt="blurry", seed=3)
        assert _run(s, "a robot arm", ["image"], **kw)["image"][0].data[:4] == b"\x89PNG"
        assert set(_run(s, "a robot arm", ["video", "audio"], **kw)) == {"video", "audio"}
        assert len(_run(s, "a robot arm", ["action"], **kw)["action"][0].data) == 16 * 32 * 4
    finally:
        s.shutdown()


def test_bagel_understanding_generation_and_cfg_parallel():
    s = _server({"model": "bagel", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["vit_encoder", "vae_encoder", "LLM", "vae_decoder"], "ranks": [0]},
                                 {"node_names": ["LLM_cfg_text"], "ranks": [1]},
                                 {"node_names": ["LLM_cfg_img", "combine_cfg"], "ranks": [2]}]})
    try:
        kw = dict(max_tokens=5, ignore_eos=True, num_steps=3, height=32, width=32, seed=1)
        assert len(_run(s, "a cat", ["text"], tensors={"image": [torch.rand(3, 32, 32)]}, **kw)["text"]) == 5
        import io

        from PIL import Image
        a = _run(s, "a cat", ["image"], **kw)
        b = _run(s, "a cat", ["image"], cfg_parallel=True, **kw)
        pa, pb = (np.asarray(Image.open(io.BytesIO(r["image"][0].data)), dtype=np.int32) for r in (a, b))
        assert np.abs(pa - pb).mean() < 4.0          # bf16: packed and three-node guidance agree closely
        _run(s, "a cat", ["image"], tensors={"image": [torch.rand(3, 32, 32)]}, cfg_img_scale=1.5, **kw)
    finally:
        s.shutdown()


def test_qwen3_omni_speech_and_tts_and_asr():
    s = _server({"model": "qwen3_omni", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["audio_encoder", "vision_encoder", "Thinker"], "ranks": [0]},
                                 {"node_names": ["Talker"], "ranks": [1]}, {"node_names": ["Code2Wav"], "ranks": [2]}]})
    try:
        res = _run(s, "say hi", ["text", "audio"], max_tokens=6, ignore_eos=True, max_audio_tokens=20,
                   tensors={"audio": [torch.randn(8000) * 0.1], "image": [torch.rand(3, 32, 32)]})
        # 20 frames of 4 samples in 4 chunks; every chunk's last causal transposed convolution gives up 2 samples
        assert len(res["text"]) == 6 and sum(len(c.data) for c in res["audio"]) == (20 * 4 - 4 * 2) * 2
    finally:
        s.shutdown()
    s = _server({"model": "qwen3_tts", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["Talker"], "ranks": [0]}, {"node_names": ["Codec"], "ranks": [1]}]})
    try:
        res = _run(s, "hello world", ["audio"], max_tokens=40, ignore_eos=True)
        assert sum(len(c.data) for c in res["audio"]) == 39 * 4 * 2
        assert s.deployment.workers[0].engines.engine_for("Talker").graph_hits >= 30
    finally:
        s.shutdown()
    for model, nodes in (("whisper_large", ["audio_encoder", "decoder"]), ("higgs_audio", ["audio_encoder", "LLM"])):
        s = _server({"model": model, "model_kwargs": {"small": True}, "node_groups": [{"node_names": nodes, "ranks": [0]}]})
        try:
            res = _run(s, "transcribe", ["text"], max_tokens=6, ignore_eos=True, tensors={"audio": [torch.randn(48000) * 0.1]})
            assert len(res["text"]) == 6
        finally:
            s.shutdown()


def test_pi05_and_vjepa2():
    s = _server({"model": "pi05", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["vit_encoder", "LLM"], "ranks": [0]}]})
    try:
        img = [torch.rand(3, 32, 32), torch.rand(3, 32, 32)]
        a = np.frombuffer(_run(s, "pick up the cup", ["action"], seed=3, tensors={"image": img})["action"][0].data, dtype=np.float32)
        b = np.frombuffer(_run(s, "pick up the cup", ["action"], seed=3, tensors={"image": img})["action"][0].data, dtype=np.float32)
        assert a.shape == (8 * 32,) and np.isfinite(a).all() and np.allclose(a, b, atol=1e-3)
    finally:
        s.shutdown()
    s = _server({"model": "vjepa2_ac", "model_kwargs": {"small": True},
                 "node_groups": [{"node_names": ["video_encoder", "predictor"], "ranks": [0]}]})
    try:
        vid = torch.rand(3, 4, 32, 32)
        _run(s, None, ["embeddings"], task="predict", seed=1, tensors={"video": [vid]})
        ro = _run(s, None, ["embeddings"], task="rollout", horizon=3,
                  tensors={"video": [vid], "actions": [torch.randn(3, 7)], "state": [torch.randn(7)]})
        assert len(ro["embeddings"]) >= 1
        mp = _run(s, None, ["embeddings"], task="mpc",
                  tensors={"video": [vid], "image": [torch.rand(3, 32, 32)], "actions": [torch.randn(5, 2, 7)], "state": [torch.randn(7)]})
        assert np.frombuffer(mp["energy"][0].data, dtype=np.float32).shape == (5,)
    finally:
        s.shutdown()
