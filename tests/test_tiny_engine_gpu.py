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
    # oracle on the same (bf16-rounded) weights in fp32 math on the CPU
    ref = tiny.oracle_generate(model.to("cpu") if False else _cpu_copy(model), prompts, 32)
    first = sum(int(a[0] == b[0]) for a, b in zip(graph, ref))
    assert first == len(prompts)
    agree = sum(int(x == y) for a, b in zip(graph, ref) for x, y in zip(a, b)) / (32 * len(prompts))
    assert agree > 0.5, f"token agreement with the fp32 oracle {agree:.2f}"


def _cpu_copy(model):
    m = tiny.build_tiny(device="cpu", dtype=torch.float32)
    with torch.no_grad():
        for (_, a), (_, b) in zip(m.named_parameters(), model.named_parameters()):
            a.copy_(b.float().cpu())
    return m
