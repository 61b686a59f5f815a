"""Config 1: tiny Qwen-style decoder, fp32 on CPU, 4 prompts of 16-64 tokens, continuous batching with paged KV
(block 16), greedy decode of 32 tokens; the engine must reproduce the cache-free oracle token for token."""
import torch

from mstar_b200.engine.kv_store import KVCacheConfig
from mstar_b200.engine.llm_engine import LLMEngine
from mstar_b200.models import tiny


def _engine(model, max_batch=4, pages=64):
    cfg = model.cfg
    kvc = KVCacheConfig(num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                        max_seq_len=256, max_num_pages=pages, page_size=16, num_qo_heads=cfg.num_heads,
                        dtype=cfg.dtype)
    return LLMEngine(model, kvc, "cpu", max_batch=max_batch, max_prefill_tokens=128)


def test_tiny_matches_oracle_cpu():
    torch.manual_seed(0)
    model = tiny.build_tiny()
    prompts = tiny.synthetic_prompts()
    ref = tiny.oracle_generate(model, prompts, 32)
    eng = _engine(model)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, 32)
    out = eng.run_to_completion()
    for i in range(len(prompts)):
        assert out[f"r{i}"] == ref[i], f"request {i} diverged"
    assert eng.cache.alloc.num_free_pages == 64          # every page came back
    assert eng.stats["prefill_tokens"] == sum(len(p) for p in prompts)


def test_continuous_batching_more_requests_than_rows():
    model = tiny.build_tiny()
    prompts = tiny.synthetic_prompts(n=5, lo=8, hi=24, seed=3)
    ref = tiny.oracle_generate(model, prompts, 6)
    eng = _engine(model, max_batch=2)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, 6)
    out = eng.run_to_completion()
    assert [out[f"r{i}"] for i in range(5)] == ref


def test_preemption_when_pool_is_small():
    model = tiny.build_tiny()
    prompts = tiny.synthetic_prompts(n=3, lo=30, hi=32, seed=5)
    ref = tiny.oracle_generate(model, prompts, 20)
    eng = _engine(model, max_batch=3, pages=8)      # 8 pages x 16 tokens < 3 x 52 tokens
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, 20)
    out = eng.run_to_completion()
    assert [out[f"r{i}"] for i in range(3)] == ref


def test_folded_norms_generate_the_same_tokens():
    """Norm gains folded into the next projection, residual add and sum of squares in the previous one: the decode
    path without norm kernels reproduces the oracle of the ORIGINAL weights token for token (fp32, CPU: the PyTorch
    statement of the fused epilogues)."""
    torch.manual_seed(0)
    model = tiny.build_tiny()
    for layer in model.layers:                      # non-trivial gains, so that folding them matters
        layer.input_layernorm.data.uniform_(0.5, 1.5)
        layer.post_attention_layernorm.data.uniform_(0.5, 1.5)
    prompts = tiny.synthetic_prompts()
    ref = tiny.oracle_generate(model, prompts, 24)
    model.fold_norms()
    assert model._norms_folded and float(model.layers[0].input_layernorm.min()) == 1.0
    eng = _engine(model)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, 24)
    out = eng.run_to_completion()
    assert [out[f"r{i}"] for i in range(len(prompts))] == ref
    assert float(model._ss.abs().sum()) > 0         # the folded path ran (its accumulators were used)
