"""Weight layouts of the projection op: the tile-packed form used by weight-streaming GEMMs."""
import pytest
import torch

from mstar_b200.ops import gemm


@pytest.mark.parametrize("N,K", [(300, 200), (128, 64), (1, 8), (257, 520)])
def test_packed_weight_round_trip_and_cpu_linear(N, K):
    g = torch.Generator().manual_seed(N)
    w = torch.randn(N, K, generator=g).bfloat16()
    pw = gemm.pack_weight(w)
    assert pw.shape == (N, K) and pw.data.shape[1] == 64 and pw.data.shape[0] % 128 == 0
    assert torch.equal(pw.unpack(), w)
    x = torch.randn(5, K, generator=g).bfloat16()
    assert torch.equal(gemm.linear(x, pw), gemm.linear(x, w))


def test_decoder_pack_weights_is_a_no_op_on_cpu():
    from mstar_b200.models import tiny
    m = tiny.build_tiny()
    m.pack_weights()
    assert isinstance(m.layers[0].self_attn.qkv_proj, torch.Tensor)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(64, 3072, 1024), (7, 1000, 520), (300, 512, 768), (2048, 1024, 512)])
def test_packed_weight_matches_plain_on_gpu(M, N, K):
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, K, generator=g) * 0.3).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    y0 = gemm.linear(x, w)
    y1 = gemm.linear(x, gemm.pack_weight(w))
    assert torch.equal(y0, y1)


@pytest.mark.gpu
def test_tiny_decoder_with_packed_weights_generates_the_same_tokens():
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.engine.llm_engine import LLMEngine
    from mstar_b200.models import tiny
    dev = torch.device("cuda", 0)
    outs = []
    for packed in (False, True):
        model = tiny.build_tiny(device=dev, dtype=torch.bfloat16)
        if packed:
            model.pack_weights()
            assert isinstance(model.layers[0].self_attn.qkv_proj, gemm.PackedWeight)
        cfg = model.cfg
        kvc = KVCacheConfig(num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            max_seq_len=256, max_num_pages=64, page_size=16, num_qo_heads=cfg.num_heads)
        eng = LLMEngine(model, kvc, dev, max_batch=4, max_prefill_tokens=256)
        for i, p in enumerate(tiny.synthetic_prompts()):
            eng.add_request(f"s{i}", p, 8)
        outs.append(eng.run_to_completion())
    assert outs[0] == outs[1]
