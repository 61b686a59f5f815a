"""Checkpoint-format loaders: strictness, and numerical parity with the reference project's own modules on shared
weights (the reference package, when installed under ``baseline/_ref``, is imported on the CPU as the oracle)."""
import os
import sys

import pytest
import torch
from safetensors.torch import save_file

from mstar_b200.models import checkpoints as ck
from mstar_b200.models.dit import AdaLNDiT, DiTConfig

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def _ref_modules():
    if not os.path.isdir(os.path.join(REF, "mstar")):
        pytest.skip("reference package not installed under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)


def _tiny_dit_cfg():
    return DiTConfig(hidden_size=48, num_layers=2, num_heads=2, head_dim=24, ffn_dim=64, in_channels=4,
                     out_channels=4, text_dim=16, text_len=8, dtype=torch.float32)


def test_wan22_loader_is_strict_and_round_trips(tmp_path):
    cfg = _tiny_dit_cfg()
    src = AdaLNDiT(cfg).init_random(3)
    keys = ck.wan22_checkpoint_keys(src)
    assert "blocks.1.attn2.to_out.0.weight" in keys and keys["patch_embedding.weight"].dim() == 5
    d = tmp_path / "transformer"
    d.mkdir()
    save_file(keys, str(d / "diffusion_pytorch_model.safetensors"))
    dst = AdaLNDiT(cfg).init_random(4)
    assert ck.load_wan22_transformer(dst, str(d))["loaded"] == len(dict(dst.named_parameters()))
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    # a missing tensor, an unknown tensor and a wrong shape each refuse the load
    for mutate in (lambda k: k.pop("blocks.0.attn1.to_k.weight"), lambda k: k.update({"blocks.0.extra.weight": torch.zeros(1)}),
                   lambda k: k.update({"proj_out.bias": torch.zeros(3)})):
        bad = dict(keys)
        mutate(bad)
        save_file(bad, str(d / "diffusion_pytorch_model.safetensors"))
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_wan22_transformer(AdaLNDiT(cfg), str(d))


def test_wan22_dit_matches_the_reference_module_on_a_shared_checkpoint(tmp_path):
    """The reference's own ``Wan22DiT`` (fp32, CPU) and ``AdaLNDiT`` loaded from the same diffusers-named
    checkpoint give the same velocity for the same latents, per-token timesteps and text embeddings."""
    _ref_modules()
    from mstar.model.wan22.components.dit import Wan22DiT
    from mstar.model.wan22.config import Wan22Config
    from mstar.model.wan22.weight_loader import remap_checkpoint_key
    rc = Wan22Config(num_attention_heads=2, attention_head_dim=24, num_layers=2, ffn_dim=64, in_channels=4,
                     out_channels=4, text_dim=16, rope_max_seq_len=64)
    torch.manual_seed(0)
    ref = Wan22DiT(rc).float().eval()
    for p in ref.parameters():
        torch.nn.init.normal_(p, std=0.2 if p.dim() > 1 else 0.05)
    for n, p in ref.named_parameters():
        if n.endswith(("q_norm.weight", "k_norm.weight", "norm2.weight")):
            p.data.add_(1.0)
    # write the reference's weights under the checkpoint's (diffusers) names: invert its own key remap
    ours = AdaLNDiT(_tiny_dit_cfg())
    names = list(ck.wan22_checkpoint_keys(ours.init_random(0)).keys())
    native = dict(ref.named_parameters())
    sd = {k: native[remap_checkpoint_key(k)].detach().clone().contiguous() for k in names}
    assert len(sd) == len(native)
    d = tmp_path / "transformer"
    d.mkdir()
    save_file(sd, str(d / "diffusion_pytorch_model.safetensors"))
    ck.load_wan22_transformer(ours, str(d))
    B, C, F, Hh, Ww = 2, 4, 2, 4, 6
    g = torch.Generator().manual_seed(1)
    lat = torch.randn(B, C, F, Hh, Ww, generator=g)
    text = torch.randn(B, 8, 16, generator=g)
    S = F * (Hh // 2) * (Ww // 2)
    ts_frame = torch.tensor([[900.0, 0.0], [500.0, 500.0]])            # per latent frame (first frame of item 0 clean)
    ts_tok = ts_frame.repeat_interleave(S // F, dim=1)
    with torch.no_grad():
        want = ref(lat, ts_tok, text)
        ctx_kv = ours.encode_context(text.reshape(B * 8, 16))
        got = ours(lat, ts_frame, ctx_kv, [8] * B)
    err = (got - want.float()).abs().max().item()
    assert err < 2e-3 * max(1.0, want.abs().max().item()), err


def _tiny_cosmos3(seed):
    from mstar_b200.models.cosmos3 import Cosmos3Transformer
    from mstar_b200.models.decoder import DecoderConfig
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=128, qk_norm=True, mrope_sections=[2, 3, 3], has_lm_head=False, dtype=torch.float32)
    return Cosmos3Transformer(cfg, 4, action_dim=8, sound_dim=8, num_domains=3).init_random(seed)


def test_cosmos3_loader_is_strict_and_round_trips(tmp_path):
    src = _tiny_cosmos3(5)
    keys = ck.cosmos3_checkpoint_keys(src)
    assert {"layers.1.self_attn.add_k_proj.weight", "layers.0.mlp_moe_gen.up_proj.weight", "norm_moe_gen.weight",
            "layers.1.input_layernorm_moe_gen.weight", "action_proj_in.fc.weight", "audio_proj_out.bias",
            "time_embedder.linear_2.weight", "layers.0.self_attn.norm_added_q.weight"} <= set(keys)
    assert keys["action_proj_in.fc.weight"].shape == (3, 8 * 64)
    keys["lm_head.weight"] = torch.zeros(128, 64)                 # present in published files, never loaded
    d = tmp_path / "transformer"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in keys.items()}, str(d / "diffusion_pytorch_model.safetensors"))
    dst = _tiny_cosmos3(6)
    assert ck.load_cosmos3_transformer(dst, str(d))["loaded"] == len(dict(dst.named_parameters()))
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    w_in, b_in, w_out, b_out = dst.action_weights(2)
    assert torch.equal(w_in, keys["action_proj_in.fc.weight"][2].view(8, 64).t())
    for mutate in (lambda k: k.pop("layers.1.mlp_moe_gen.gate_proj.weight"),
                   lambda k: k.update({"layers.0.self_attn.to_extra.weight": torch.zeros(1)}),
                   lambda k: k.update({"audio_proj_in.weight": torch.zeros(64, 9)}),
                   lambda k: k.pop("norm_moe_gen.weight")):
        badk = dict(keys)
        mutate(badk)
        save_file({k: v.contiguous() for k, v in badk.items()}, str(d / "diffusion_pytorch_model.safetensors"))
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_cosmos3_transformer(_tiny_cosmos3(7), str(d))


def test_t5_encoder_matches_hugging_face_umt5_on_shared_weights():
    """Our T5 / UMT5 encoder, loaded from a Hugging Face state dict, reproduces ``UMT5EncoderModel`` (fp32, CPU)."""
    transformers = pytest.importorskip("transformers")
    from mstar_b200.models.encoders import T5Encoder
    cfg = transformers.UMT5Config(vocab_size=96, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4,
                                  relative_attention_num_buckets=32, relative_attention_max_distance=128,
                                  feed_forward_proj="gated-gelu", dropout_rate=0.0)
    torch.manual_seed(0)
    hf = transformers.UMT5EncoderModel(cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.copy_(torch.randn_like(p) * (0.3 if p.dim() > 1 else 0.2) + (1.0 if p.dim() == 1 else 0.0))
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    ours = T5Encoder(vocab_size=96, hidden=64, layers=2, heads=4, head_dim=16, ffn=128, buckets=32, max_distance=128,
                     per_layer_bias=True, dtype=torch.float32)
    assert ck.load_t5_encoder(ours, sd)["loaded"] == len(dict(ours.named_parameters()))
    ids = torch.randint(0, 96, (23,))
    with torch.no_grad():
        want = hf(input_ids=ids[None]).last_hidden_state[0]
    got = ours(ids)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), (got - want).abs().max()
    bad = dict(sd)
    bad.pop("encoder.block.1.layer.1.DenseReluDense.wi_1.weight")
    with pytest.raises(ck.CheckpointMismatch):
        ck.load_t5_encoder(T5Encoder(vocab_size=96, hidden=64, layers=2, heads=4, head_dim=16, ffn=128,
                                     dtype=torch.float32), bad)


def test_whisper_loaders_are_strict_and_the_encoder_matches_hugging_face():
    transformers = pytest.importorskip("transformers")
    from mstar_b200.models.encoders import AudioEncoder, EncoderConfig
    from mstar_b200.models.whisper import WhisperDecoder
    cfg = transformers.WhisperConfig(vocab_size=120, num_mel_bins=16, d_model=64, encoder_layers=2, decoder_layers=2,
                                     encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=128,
                                     decoder_ffn_dim=128, max_source_positions=40, max_target_positions=24,
                                     dropout=0.0, attention_dropout=0.0, activation_dropout=0.0, pad_token_id=0, bos_token_id=1,
                                     eos_token_id=2, decoder_start_token_id=1)
    torch.manual_seed(1)
    hf = transformers.WhisperForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "embed_positions" not in n:
                p.copy_(torch.randn_like(p) * (0.15 if p.dim() > 1 else 0.1) + (1.0 if "layer_norm.weight" in n else 0.0))
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    ec = EncoderConfig(hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_dim=128, norm="layernorm",
                       act="gelu_erf", qkv_bias=True, eps=1e-5, dtype=torch.float32)        # the checkpoint's exact GELU
    enc = AudioEncoder(ec, n_mels=16, max_frames=40)
    assert ck.load_whisper_encoder(enc, sd)["loaded"] == len(dict(enc.named_parameters()))
    mel = torch.randn(16, 80)                                   # 80 frames -> 40 positions
    with torch.no_grad():
        want = hf.model.encoder(mel[None]).last_hidden_state[0]
    got, lens = enc([mel])
    assert lens == [40]
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), (got - want).abs().max()
    dec = WhisperDecoder(vocab=120, hidden=64, layers=2, heads=4, ffn=128, max_pos=24, dtype=torch.float32)
    assert ck.load_whisper_decoder(dec, sd)["loaded"] == len(dict(dec.named_parameters()))
    assert torch.equal(dec.layers[1].ckv_w[:64], sd["model.decoder.layers.1.encoder_attn.k_proj.weight"])
    assert torch.equal(dec.layers[0].qkv_b[64:128], torch.zeros(64))            # the key projection has no bias
    for mutate in (lambda k: k.pop("model.decoder.layers.0.encoder_attn.v_proj.bias"),
                   lambda k: k.update({"model.decoder.layers.0.extra.weight": torch.zeros(1)})):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_whisper_decoder(WhisperDecoder(vocab=120, hidden=64, layers=2, heads=4, ffn=128, max_pos=24,
                                                   dtype=torch.float32), bad)


def test_siglip_vision_tower_matches_hugging_face_on_shared_weights():
    transformers = pytest.importorskip("transformers")
    from mstar_b200.models.encoders import EncoderConfig, VisionEncoder
    cfg = transformers.SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                          num_channels=3, image_size=32, patch_size=8, hidden_act="gelu_pytorch_tanh",
                                          layer_norm_eps=1e-6, attention_dropout=0.0, vision_use_head=False)
    torch.manual_seed(2)
    hf = transformers.SiglipVisionModel(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.copy_(torch.randn_like(p) * (0.15 if p.dim() > 1 else 0.1) + (1.0 if ("layer_norm" in n or "layernorm" in n) and n.endswith("weight") else 0.0))
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    ec = EncoderConfig(hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_dim=128, norm="layernorm", act="gelu",
                       qkv_bias=True, eps=1e-6, dtype=torch.float32)
    enc = VisionEncoder(ec, patch=8, pos="learned", pos_grid=4)
    assert ck.load_siglip_vision(enc, sd)["loaded"] == len(dict(enc.named_parameters()))
    img = torch.randn(3, 32, 32)
    with torch.no_grad():
        want = hf(pixel_values=img[None]).last_hidden_state[0]
    got, lens, grids = enc([img])
    assert lens == [16] and grids == [(1, 4, 4)]
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), (got - want).abs().max()
    bad = dict(sd)
    bad.pop("vision_model.encoder.layers.1.mlp.fc2.bias")
    with pytest.raises(ck.CheckpointMismatch):
        ck.load_siglip_vision(VisionEncoder(ec, patch=8, pos="learned", pos_grid=4), bad)


def test_bagel_loader_round_trips_the_published_layout_and_is_strict():
    from mstar_b200.models.bagel import BagelMoT
    from mstar_b200.models.decoder import DecoderConfig
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=128, qkv_bias=True, qk_norm=True, dtype=torch.float32)
    src = BagelMoT(cfg, 8).init_random(1)
    keys = ck.bagel_checkpoint_keys(src)
    assert {"language_model.model.layers.1.self_attn.k_proj_moe_gen.bias", "language_model.model.norm_moe_gen.weight",
            "language_model.model.layers.0.mlp_moe_gen.up_proj.weight", "time_embedder.mlp.2.weight",
            "language_model.model.layers.1.self_attn.q_norm_moe_gen.weight", "vae2llm.weight"} <= set(keys)
    # what other nodes load, and the frozen sine-cosine tables, are accepted and skipped
    keys.update({"latent_pos_embed.pos_embed": torch.zeros(16, 64), "vit_model.vision_model.post_layernorm.weight": torch.ones(8),
                 "connector.fc1.weight": torch.zeros(4, 4), "vit_pos_embed.pos_embed": torch.zeros(4, 4)})
    dst = BagelMoT(cfg, 8).init_random(2)
    assert ck.load_bagel_mot(dst, keys)["loaded"] == len(dict(dst.named_parameters()))
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    for mutate in (lambda k: k.pop("language_model.model.layers.0.self_attn.v_proj_moe_gen.bias"),
                   lambda k: k.update({"language_model.model.layers.0.mlp_moe_gen.extra.weight": torch.zeros(1)}),
                   lambda k: k.update({"llm2vae.weight": torch.zeros(8, 63)})):
        bad = dict(keys)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_bagel_mot(BagelMoT(cfg, 8), bad)


def test_bagel_vision_tower_and_connector_load_from_the_published_names(tmp_path):
    transformers = pytest.importorskip("transformers")
    from mstar_b200.models.bagel import BagelModel
    m = BagelModel(model_dir=str(tmp_path), skip_weight_loading=False, small=True)
    c = m.vit_cfg
    hf_cfg = transformers.SiglipVisionConfig(hidden_size=c.hidden_size, intermediate_size=c.ffn_dim,
                                             num_hidden_layers=c.num_layers, num_attention_heads=c.num_heads, num_channels=3,
                                             image_size=m.vit_patch * 8, patch_size=m.vit_patch, vision_use_head=False)
    torch.manual_seed(4)
    hf = transformers.SiglipVisionModel(hf_cfg).float()
    H, out = c.hidden_size, m.cfg.hidden_size
    keys = {"vit_model." + k: v.detach().clone() for k, v in hf.state_dict().items()}
    keys.update({"connector.fc1.weight": torch.randn(H, H), "connector.fc1.bias": torch.randn(H),
                 "connector.fc2.weight": torch.randn(out, H), "connector.fc2.bias": torch.randn(out),
                 "vit_pos_embed.pos_embed": torch.randn(64, H), "llm2vae.bias": torch.zeros(3)})
    save_file({k: v.contiguous() for k, v in keys.items()}, str(tmp_path / "ema.safetensors"))
    sub = m.get_submodule("vit_encoder", "cpu")
    enc = sub.enc
    assert torch.allclose(enc.proj2_w.float(), keys["connector.fc2.weight"], atol=1e-2)
    assert torch.allclose(enc.pos_table.float(), keys["vit_pos_embed.pos_embed"], atol=1e-2)
    q = keys["vit_model.vision_model.encoder.layers.0.self_attn.q_proj.weight"]
    assert torch.allclose(enc.enc.layers[0].qkv_w[:q.shape[0]].float(), q, atol=1e-2)
    keys.pop("connector.fc2.bias")
    save_file({k: v.contiguous() for k, v in keys.items()}, str(tmp_path / "ema.safetensors"))
    with pytest.raises(ck.CheckpointMismatch):
        m.get_submodule("vit_encoder", "cpu")


def test_image_autoencoder_matches_the_reference_module_on_a_shared_checkpoint():
    """The reference's own ``BagelAutoEncoder`` (fp32, CPU) and ``ConvVAE`` loaded from its state dict (the
    ``ae.safetensors`` names) encode and decode to the same tensors; a missing, extra or mis-shaped tensor raises."""
    _ref_modules()
    from mstar.model.bagel.components.autoencoder import BagelAutoEncoder
    from mstar.model.bagel.config import BagelAutoEncoderConfig
    from mstar_b200.models.vae import ConvVAE, VAEConfig
    torch.manual_seed(0)
    rc = BagelAutoEncoderConfig(resolution=32, ch=32, ch_mult=(1, 2, 2), num_res_blocks=1, z_channels=4)
    ref = BagelAutoEncoder(rc).float().eval()
    ref.reg.sample = False
    for n, p in ref.named_parameters():
        torch.nn.init.normal_(p, std=0.08 if p.dim() > 1 else 0.05)
        if "norm" in n and n.endswith("weight"):
            p.data.add_(1.0)
    sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    cfg = VAEConfig(dims=2, latent_channels=4, base_channels=32, channel_mult=(1, 2, 2), num_res_blocks=1,
                    scaling_factor=rc.scale_factor, shift_factor=rc.shift_factor)
    ours = ConvVAE(cfg).float().eval()
    ck.load_image_autoencoder(ours, sd)
    x = torch.rand(2, 3, 32, 48) * 2 - 1
    with torch.no_grad():
        z_ref, z = ref.encode(x), ours.encode(x)
        assert z.shape == z_ref.shape == (2, 4, 8, 12)
        assert (z - z_ref).abs().max().item() < 1e-4 * max(1.0, z_ref.abs().max().item())
        px_ref, px = ref.decode(z_ref).clamp(-1, 1), ours.decode(z_ref)
        assert (px - px_ref).abs().max().item() < 1e-4
    for mutate in (lambda d: d.pop("decoder.up.1.upsample.conv.weight"),
                   lambda d: d.update({"encoder.down.0.attn.0.norm.weight": torch.zeros(32)}),
                   lambda d: d.update({"encoder.mid.attn_1.q.weight": torch.zeros(64, 32, 1, 1)})):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_image_autoencoder(ConvVAE(cfg), bad)


def test_wan22_loader_fills_a_tensor_parallel_model_with_its_shards(tmp_path):
    """Every rank of a tensor-parallel ``AdaLNDiT`` gets, from the diffusers-named checkpoint, exactly the slices of
    the single-rank model's parameters that ``adaln_shard`` names (whole heads of q, k and v; MLP columns)."""
    from mstar_b200.models.dit import adaln_shard
    from mstar_b200.parallel.comm import CommGroup
    cfg = _tiny_dit_cfg()
    one = AdaLNDiT(cfg).init_random(3)
    d = tmp_path / "transformer"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in ck.wan22_checkpoint_keys(one).items()}, str(d / "diffusion_pytorch_model.safetensors"))
    full = dict(one.named_parameters())
    for rank in range(2):
        tp = CommGroup(None, [0, 1], rank)
        two = AdaLNDiT(cfg, tp=tp)
        ck.load_wan22_transformer(two, str(d))
        for n, p in two.named_parameters():
            assert torch.equal(p, adaln_shard(n, full[n], rank, 2)), n
        A = cfg.num_heads * cfg.head_dim // 2
        assert two.blocks[0].qkv_w.shape[0] == 3 * A
        assert torch.equal(two.blocks[0].qkv_w[A:2 * A], full["blocks.0.qkv_w"][2 * A + rank * A:2 * A + (rank + 1) * A])
