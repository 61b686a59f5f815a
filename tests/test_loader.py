"""Checkpoint loader: a Hugging Face-style safetensors checkpoint written from a reference model must load into
single-rank and tensor-parallel decoders that compute the same logits."""
import torch

from mstar_b200.engine.cache_manager import BatchedCacheManager
from mstar_b200.engine.kv_store import KVCacheConfig
from mstar_b200.models.decoder import DecoderConfig, DecoderLM
from mstar_b200.models.loader import iter_safetensors, load_decoder_from_hf, load_named_tensors


def _write_hf(tmp, cfg, seed=0, moe=False):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    H, D, Hq, Hkv, F = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size
    r = lambda *s: torch.randn(s, generator=g) * 0.05  # noqa: E731
    sd = {"model.embed_tokens.weight": r(cfg.vocab_size, H), "model.norm.weight": 1 + r(H), "lm_head.weight": r(cfg.vocab_size, H)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": r(Hq * D, H), p + "self_attn.k_proj.weight": r(Hkv * D, H),
                   p + "self_attn.v_proj.weight": r(Hkv * D, H), p + "self_attn.o_proj.weight": r(H, Hq * D),
                   p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H)})
        if moe:
            sd[p + "mlp.gate.weight"] = r(cfg.num_experts, H)
            for e in range(cfg.num_experts):
                q = p + f"mlp.experts.{e}."
                I = cfg.moe_intermediate_size
                sd.update({q + "gate_proj.weight": r(I, H), q + "up_proj.weight": r(I, H), q + "down_proj.weight": r(H, I)})
        else:
            sd.update({p + "mlp.gate_proj.weight": r(F, H), p + "mlp.up_proj.weight": r(F, H), p + "mlp.down_proj.weight": r(H, F)})
    keys = sorted(sd)
    save_file({k: sd[k].contiguous() for k in keys[::2]}, str(tmp / "model-00001.safetensors"))
    save_file({k: sd[k].contiguous() for k in keys[1::2]}, str(tmp / "model-00002.safetensors"))
    return sd


def _logits(lm, cfg, ids, kvh):
    kvc = KVCacheConfig(cfg.num_layers, kvh, cfg.head_dim, max_seq_len=64, max_num_pages=8, page_size=16,
                        num_qo_heads=cfg.num_heads, dtype=torch.float32)
    cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64)
    cm.add_request("r")
    return lm(cm.plan(["r"], [ids.numel()]), input_ids=ids)


def test_dense_checkpoint_loads_and_matches_manual_forward(tmp_path):
    cfg = DecoderConfig(hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8, intermediate_size=64,
                        vocab_size=50, dtype=torch.float32)
    sd = _write_hf(tmp_path, cfg)
    assert len(list(iter_safetensors(str(tmp_path)))) == len(sd)
    lm = DecoderLM(cfg)
    info = load_decoder_from_hf(lm, str(tmp_path))
    assert not info["incomplete"] and info["loaded"] > 10
    ids = torch.arange(7)
    out = _logits(lm, cfg, ids, 2)
    # an independent restatement of the first layer's q projection: fused rows [q | k | v]
    assert torch.equal(lm.layers[0].self_attn.qkv_proj[:32], sd["model.layers.0.self_attn.q_proj.weight"])
    assert torch.equal(lm.layers[1].mlp.gate_up_proj[0::2], sd["model.layers.1.mlp.gate_proj.weight"])
    assert out.shape == (1, 50) and torch.isfinite(out).all()


def test_moe_checkpoint_stacks_experts(tmp_path):
    cfg = DecoderConfig(hidden_size=32, num_layers=1, num_heads=4, num_kv_heads=2, head_dim=8, intermediate_size=64,
                        vocab_size=50, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, dtype=torch.float32)
    sd = _write_hf(tmp_path, cfg, moe=True)
    lm = DecoderLM(cfg)
    info = load_decoder_from_hf(lm, str(tmp_path))
    assert not info["incomplete"]
    assert torch.equal(lm.layers[0].mlp.w2[3], sd["model.layers.0.mlp.experts.3.down_proj.weight"])
    assert torch.equal(lm.layers[0].mlp.w13[2][1::2], sd["model.layers.0.mlp.experts.2.up_proj.weight"])
    assert torch.equal(lm.layers[0].mlp.router, sd["model.layers.0.mlp.gate.weight"])


def test_named_tensor_loader_reports_mismatches(tmp_path):
    from safetensors.torch import save_file
    m = torch.nn.Linear(4, 3)
    save_file({"weight": torch.ones(3, 4), "extra": torch.zeros(2)}, str(tmp_path / "model.safetensors"))
    rep = load_named_tensors(m, str(tmp_path))
    assert rep["missing"] == ["bias"] and rep["unexpected"] == ["extra"] and torch.equal(m.weight.data, torch.ones(3, 4))


def test_decoder_loader_is_strict_and_ties_a_missing_head(tmp_path):
    import pytest
    from safetensors.torch import save_file
    from mstar_b200.models.checkpoints import CheckpointMismatch
    cfg = DecoderConfig(hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8, intermediate_size=64,
                        vocab_size=50, dtype=torch.float32)
    sd = _write_hf(tmp_path, cfg)
    for f in tmp_path.iterdir():
        f.unlink()
    for mutate in (lambda d: d.pop("model.layers.1.post_attention_layernorm.weight"),          # a parameter stays unloaded
                   lambda d: d.update({"model.layers.0.self_attn.rotary.weight": torch.zeros(2)}),  # a tensor finds no home
                   lambda d: d.pop("model.layers.0.mlp.up_proj.weight")):                          # half of a fused group
        bad = dict(sd)
        mutate(bad)
        d = tmp_path / f"bad{len(list(tmp_path.iterdir()))}"
        d.mkdir()
        save_file({k: v.contiguous() for k, v in bad.items()}, str(d / "model.safetensors"))
        with pytest.raises(CheckpointMismatch):
            load_decoder_from_hf(DecoderLM(cfg), str(d))
        info = load_decoder_from_hf(DecoderLM(cfg), str(d), strict=False)
        assert info["missing"] or info["unused"] or info["incomplete"]
    tied = {k: v for k, v in sd.items() if k != "lm_head.weight"}
    tied["model.rotary_emb.inv_freq"] = torch.zeros(4)                  # old checkpoints carry this buffer: ignored
    d = tmp_path / "tied"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in tied.items()}, str(d / "model.safetensors"))
    lm = DecoderLM(cfg)
    info = load_decoder_from_hf(lm, str(d))
    assert not info["missing"] and torch.equal(lm.lm_head, lm.embed_tokens)


def test_llama3_rope_scaled_decoder_matches_hugging_face_llama(tmp_path):
    """The Orpheus backbone's layout at test size (grouped KV heads, head_dim x heads != hidden, tied head, Llama-3
    frequency-dependent rotary scaling) loaded from Hugging Face names against ``transformers.LlamaModel``."""
    import pytest
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import save_file
    scaling = dict(factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    hc = transformers.LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5,
                                  tie_word_embeddings=True, attention_bias=False, max_position_embeddings=512,
                                  rope_parameters=dict(rope_type="llama3", rope_theta=500000.0, **scaling))
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.1)
        if "norm" in n:
            p.data.add_(1.0)
    sd = {k: v.detach().clone().contiguous() for k, v in hf.state_dict().items() if k != "lm_head.weight"}
    save_file(sd, str(tmp_path / "model.safetensors"))
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=96,
                        vocab_size=300, rms_eps=1e-5, rope_theta=500000.0, rope_llama3=scaling, tie_embeddings=True,
                        dtype=torch.float32)
    lm = DecoderLM(cfg)
    assert not load_decoder_from_hf(lm, str(tmp_path))["missing"]
    T = 100                                              # past the original context length: every band of the scaling
    ids = torch.randint(0, 300, (T,), generator=torch.Generator().manual_seed(1))
    kvc = KVCacheConfig(2, 2, 32, max_seq_len=256, max_num_pages=16, page_size=16, num_qo_heads=4, dtype=torch.float32)
    cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=256)
    cm.add_request("r")
    with torch.no_grad():
        want = hf(input_ids=ids[None]).logits[0]
        got = lm(cm.plan(["r"], [T], group=2), input_ids=ids, all_logits=True)
    assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_qwen2_style_decoder_with_qkv_bias_matches_hugging_face(tmp_path):
    """Fused q / k / v biases and untied head (the layout of BAGEL's understanding expert and of Qwen2.5 backbones)
    against ``transformers.Qwen2ForCausalLM``."""
    import pytest
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import save_file
    hc = transformers.Qwen2Config(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                  max_position_embeddings=256, use_sliding_window=False,
                                  rope_parameters=dict(rope_type="default", rope_theta=1e6))
    torch.manual_seed(0)
    hf = transformers.Qwen2ForCausalLM(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.1)
        if "norm" in n:
            p.data.add_(1.0)
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()}, str(tmp_path / "model.safetensors"))
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=200, rms_eps=1e-6, rope_theta=1e6, qkv_bias=True, dtype=torch.float32)
    lm = DecoderLM(cfg)
    assert not load_decoder_from_hf(lm, str(tmp_path))["missing"]
    ids = torch.randint(0, 200, (23,), generator=torch.Generator().manual_seed(1))
    kvc = KVCacheConfig(2, 2, 16, max_seq_len=64, max_num_pages=8, page_size=16, num_qo_heads=4, dtype=torch.float32)
    cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64)
    cm.add_request("r")
    with torch.no_grad():
        want = hf(input_ids=ids[None]).logits[0]
        got = lm(cm.plan(["r"], [23], group=2), input_ids=ids, all_logits=True)
    assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
