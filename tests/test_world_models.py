"""Policy / world models on CPU through the serving stack: Pi0.5-class action chunks, V-JEPA 2(-AC) prediction,
rollout and planning scores; piecewise graph runner bookkeeping."""
import numpy as np
import pytest
import torch

from mstar_b200.api_server.server import APIServer
from mstar_b200.engine.piecewise_graph import PiecewiseCudaGraphRunner, signature


def test_piecewise_runner_signatures_and_cpu_passthrough():
    r = PiecewiseCudaGraphRunner(enabled=True)        # no GPU here: pieces run eagerly
    a, b = torch.ones(3, 4), torch.ones(5, 4)
    assert signature("blk", [a]) != signature("blk", [b]) and signature("blk", [a]) == signature("blk", [a.clone()])
    assert torch.equal(r.run("blk", lambda x: x * 2, a), a * 2)
    assert r.stats["eager"] == 1 and r.stats["captures"] == 0


def test_pi05_action_chunk_is_seeded_and_depends_on_the_observation():
    cfg = {"model": "pi05", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["vit_encoder"], "ranks": [0]}, {"node_names": ["LLM"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        img = [torch.rand(3, 16, 16), torch.rand(3, 16, 16)]

        def act(images, prompt="pick up the cup"):
            rid = s.submit_request(prompt, output_modalities=["action"], model_kwargs=dict(seed=3, state=[0.1, -0.5]),
                                   tensors={"image": images})
            res = s.collect_results(rid, 120)
            assert "error" not in res, res
            return np.frombuffer(res["action"][0].data, dtype=np.float32).reshape(8, 32)
        a, b, c = act(img), act(img), act([img[1], img[0]])
        assert np.allclose(a, b) and not np.allclose(a, c) and np.isfinite(a).all()
        eng = s.deployment.workers[1].engines.engine_for("LLM")
        import time
        for _ in range(100):          # the teardown message reaches the worker after the client has its result
            if eng.cache.alloc.num_free_pages == eng.cache.alloc.total_pages:
                break
            time.sleep(0.02)
        assert eng.cache.alloc.num_free_pages == eng.cache.alloc.total_pages
    finally:
        s.shutdown()


@pytest.fixture(scope="module")
def vjepa_server():
    cfg = {"model": "vjepa2_ac", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["video_encoder"], "ranks": [0]}, {"node_names": ["predictor"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def test_vjepa2_predict_encode_rollout_and_planning(vjepa_server):
    s = vjepa_server
    vid = torch.rand(3, 4, 16, 16)         # 2 tubelet frames x 4 x 4 patches = 32 tokens of width 32

    def run(mk, tens):
        res = s.collect_results(s.submit_request(None, output_modalities=["embeddings"], model_kwargs=mk, tensors=tens), 120)
        assert "error" not in res, res
        return res
    assert len(run(dict(task="predict", seed=1), {"video": [vid]})["embeddings"][0].data) == 16 * 32 * 4
    assert len(run(dict(task="encode"), {"video": [vid]})["embeddings"][0].data) == 32 * 32 * 4
    ro = run(dict(task="rollout", horizon=3), {"video": [vid], "actions": [torch.randn(3, 7)], "state": [torch.randn(7)]})
    assert sum(len(c.data) for c in ro["embeddings"]) == 3 * 16 * 32 * 4
    acts = torch.randn(5, 2, 7)
    mp = run(dict(task="mpc"), {"video": [vid], "image": [torch.rand(3, 16, 16)], "actions": [acts], "state": [torch.randn(7)]})
    e = np.frombuffer(mp["energy"][0].data, dtype=np.float32)
    best = np.frombuffer(mp["action"][0].data, dtype=np.float32).reshape(2, 7)
    assert e.shape == (5,) and np.allclose(best, acts[int(e.argmin())].numpy())
