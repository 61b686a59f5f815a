"""Tiny decoder on the GPU through the real kernels: eager == CUDA graph, and agreement with the fp32 oracle."""
import pytest
import torch

from mstar_b200.engine.kv_store import KVCacheConfig
from mstar_b200.engine.llm_engine import LLMEngine
from mstar_b200.models import tiny

pytestmark = pytest.mark.gpu


def _run(model, prompts, n, graphs, max_batch=4):
    cfg = model.cfg
    kvc = KVCacheConfig(num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                        max_seq_len=256, max_num_pages=64, page_size=16, num_qo_heads=cfg.num_heads)
    eng = LLMEngine(model, kvc, "cuda", max_batch=max_batch, max_prefill_tokens=256, use_cuda_graphs=graphs)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, n)
    out = eng.run_to_completion()
    torch.cuda.synchronize()
    eng.check_status()
    return [out[f"r{i}"] for i in range(len(prompts))], eng


def test_tiny_gpu_graph_equals_eager_and_tracks_oracle():
    model = tiny.build_tiny(device="cuda", dtype=torch.bfloat16)
    prompts = tiny.synthetic_prompts()
    eager, _ = _run(model, prompts, 32, graphs=False)
    graph, eng = _run(model, prompts, 32, graphs=True)
    assert eager == graph
    assert eng.stats["graph_replays"] > 0 and eng.launches_per_decode_graph
    # oracle on the same (bf16-rounded) weights in fp32 math on the CPU, teacher-forced along the GPU's tokens: every
    # token must be the oracle's argmax or a near tie within the bf16 error of the logits
    bad, exact = tiny.oracle_violations(tiny.fp32_copy(model), prompts, graph, rel_tol=2e-2)
    assert not bad, f"tokens outside the oracle's tolerance: {bad[:5]}"
    assert all(g[0] == r[0] for g, r in zip(graph, tiny.oracle_generate(tiny.fp32_copy(model), prompts, 1)))
    assert exact > 0.9, f"only {exact:.2f} of the tokens are the oracle's exact argmax"


def test_tiny_served_on_the_gpu_tracks_the_oracle():
    """The serving stack (API server core, conductor, worker, KV engine with decode graphs and speculative bursts)
    on the GPU gives the oracle's tokens for the tiny model."""
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "tiny", "model_kwargs": {"dtype": "bfloat16", "page_size": 16, "max_num_pages": 128},
           "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        prompts = tiny.synthetic_prompts()
        rids = [s.submit_request(" ".join(map(str, p)), model_kwargs=dict(max_tokens=24, temperature=0.0, ignore_eos=True))
                for p in prompts]
        gens = []
        for r in rids:
            res = s.collect_results(r, 120)
            assert "error" not in res, res.get("error")
            gens.append([int(t) for t in b"".join(c.data for c in res["text"]).decode().split()])
        w = s.deployment.workers[0]
        eng = w.engines.engine_for("LLM")
        lm = eng.submodules["LLM"].lm
        assert eng.graph_hits > 0 and all(len(g) == 24 for g in gens)
        bad, exact = tiny.oracle_violations(tiny.fp32_copy(lm), prompts, gens, rel_tol=2e-2)
        assert not bad, bad[:5]
        assert exact > 0.9
    finally:
        s.shutdown()
