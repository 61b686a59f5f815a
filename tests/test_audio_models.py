"""Speech models on CPU: Whisper-class decoder consistency (prefill + decode == longer prefill, cross-attention pool
slots), and the models through the serving stack with test-sized weights."""
import pytest
import torch

from mstar_b200.engine.cache_manager import BatchedCacheManager
from mstar_b200.engine.kv_store import KVCacheConfig


def test_whisper_decoder_incremental_equals_full_and_slots_are_independent():
    from mstar_b200.models.whisper import CrossAttnPool, WhisperDecoder
    dec = WhisperDecoder(vocab=300, hidden=64, layers=2, heads=4, ffn=128, dtype=torch.float32).init_random(1)
    for L in dec.layers:           # non-trivial biases
        L.qkv_b.data.normal_(0, 0.1)
        L.ckv_b.data.normal_(0, 0.1)
    pool = CrossAttnPool(2, 8, 40, 4, 16, torch.float32, "cpu")
    g = torch.Generator().manual_seed(0)
    feats = {"a": torch.randn(33, 64, generator=g), "b": torch.randn(17, 64, generator=g)}
    slots = {"a": 5, "b": 2}
    for r in feats:
        dec.project_cross(feats[r], pool, slots[r])
    ids = {"a": torch.randint(0, 300, (7,), generator=g), "b": torch.randint(0, 300, (4,), generator=g)}

    def fresh():
        kvc = KVCacheConfig(2, 4, 16, max_seq_len=64, max_num_pages=16, page_size=8, num_qo_heads=4, dtype=torch.float32)
        return BatchedCacheManager(kvc, "cpu", max_batch=4, max_tokens=64)
    # full prefill of both requests in one batch
    cm = fresh()
    ctx = cm.plan(["a", "b"], [7, 4], row_slots=[5, 2])
    full = dec(ctx, torch.cat([ids["a"], ids["b"]]), pool)
    # prefill without the last token, then one batched decode step
    cm = fresh()
    ctx = cm.plan(["a", "b"], [6, 3], row_slots=[5, 2])
    dec(ctx, torch.cat([ids["a"][:6], ids["b"][:3]]), pool)
    cm.advance_seq_lens(ctx)
    ctx = cm.plan(["b", "a"], [1, 1], row_slots=[2, 5])               # other order: slots, not rows, pick the audio
    step = dec(ctx, torch.stack([ids["b"][3], ids["a"][6]]), pool)
    assert (step[1] - full[0]).abs().max().item() < 1e-4
    assert (step[0] - full[1]).abs().max().item() < 1e-4
    # a request alone gives the same logits as inside the batch
    cm = fresh()
    solo = dec(cm.plan(["b"], [4], row_slots=[2]), ids["b"], pool)
    assert (solo[0] - full[1]).abs().max().item() < 1e-4


@pytest.fixture(scope="module")
def whisper_server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "whisper_large", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["audio_encoder"], "ranks": [0]}, {"node_names": ["decoder"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def test_whisper_serving_two_requests(whisper_server):
    rids = [whisper_server.submit_request(None, output_modalities=["text"], model_kwargs=dict(max_tokens=5),
                                          tensors={"audio": [torch.randn(16000 * (i + 1)) * 0.1]}) for i in range(2)]
    for rid in rids:
        res = whisper_server.collect_results(rid, 120)
        assert "error" not in res and len(res["text"]) == 5
