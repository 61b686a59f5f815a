"""Higgs-Audio in the published layout: audio front end against Whisper's feature extractor, tower + projector against
the reference's modules on shared weights, decoder names, placeholder counts."""
import pytest
import torch

from conftest import reference_module


def test_log_mel_matches_whisper_feature_extractor():
    from transformers import WhisperFeatureExtractor
    from mstar_b200.models.encoders import log_mel_spectrogram
    g = torch.Generator().manual_seed(0)
    for n_mels, n in ((80, 48000), (128, 64000), (128, 30000)):
        wav = (torch.randn(n, generator=g) * 0.1).clamp(-1, 1)
        fe = WhisperFeatureExtractor(feature_size=n_mels)
        ref = fe([wav.numpy()], sampling_rate=16000, padding="longest", truncation=False, return_tensors="pt")
        got = log_mel_spectrogram(wav, n_mels=n_mels)
        assert got.shape == ref["input_features"][0].shape
        assert (got - ref["input_features"][0]).abs().max() < 1e-4


def _reference_pair():
    cfg_mod = reference_module("mstar.model.higgs_audio.config")
    tower_mod = reference_module("mstar.model.higgs_audio.components.audio_tower")
    cfg = cfg_mod.HiggsAudioModelConfig(hidden_size=48, audio_d_model=32, audio_encoder_layers=2,
                                        audio_encoder_attention_heads=2, audio_encoder_ffn_dim=64,
                                        audio_num_mel_bins=16, audio_max_source_positions=1500)
    torch.manual_seed(0)
    tower, proj = tower_mod.HiggsAudioTower(cfg).eval(), tower_mod.HiggsAudioFeatureProjector(cfg).eval()
    with torch.no_grad():
        for p in list(tower.parameters()) + list(proj.parameters()):
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = {f"audio_tower.{k}": v for k, v in tower.state_dict().items()}
    sd.update({f"audio_encoder_proj.{k}": v for k, v in proj.state_dict().items()})
    return cfg, tower, proj, sd


def _ours(sd):
    from mstar_b200.models.checkpoints import load_higgs_audio_tower
    from mstar_b200.models.encoders import AudioEncoder, EncoderConfig
    from mstar_b200.models.higgs_audio import AudioProjector
    c = EncoderConfig(32, 2, 2, 16, 64, act="gelu_erf", eps=1e-5, dtype=torch.float32)
    enc = AudioEncoder(c, n_mels=16, max_frames=1500, pool=2)
    proj = AudioProjector(32, 2048, 48, torch.float32, "cpu")
    res = load_higgs_audio_tower(enc, proj, sd)
    return enc, proj, res


def test_tower_and_projector_match_the_reference_modules():
    cfg, tower, rproj, sd = _reference_pair()
    enc, proj, res = _ours(sd)
    assert res["tower"]["loaded"] > 0 and res["projector"]["loaded"] == 6
    g = torch.Generator().manual_seed(1)
    mels = torch.randn(3, 16, 400, generator=g)
    with torch.no_grad():
        want = rproj(tower(mels))                                    # [3, 50, 48]
        feats, lens = enc(list(mels))
        got, rows = proj(feats, lens)
    assert lens == [100] * 3 and rows == [50] * 3 and want.shape == (3, 50, 48)
    assert (got.reshape(3, 50, 48) - want).abs().max() < 2e-4
    # an odd frame count: the pooling drops the remainder, the projector convolution rounds up
    with torch.no_grad():
        want = rproj(tower(mels[:1, :, :298]))
        feats, lens = enc([mels[0, :, :298]])
        got, rows = proj(feats, lens)
    assert rows == [want.shape[1]] and (got - want[0]).abs().max() < 2e-4
    assert cfg.encoder_output_length(298) == rows[0]


def test_loader_is_strict():
    from mstar_b200.models.checkpoints import CheckpointMismatch
    _, _, _, sd = _reference_pair()
    missing = {k: v for k, v in sd.items() if k != "audio_encoder_proj.linear2.bias"}
    with pytest.raises(CheckpointMismatch):
        _ours(missing)
    extra = dict(sd)
    extra["audio_tower.layers.0.extra.weight"] = torch.zeros(2)
    with pytest.raises(CheckpointMismatch):
        _ours(extra)


def test_rows_and_decoder_names():
    from mstar_b200.models import higgs_audio as H
    cfg_mod = reference_module("mstar.model.higgs_audio.config")
    ref = cfg_mod.HiggsAudioModelConfig()
    for n in (1600, 16000, 48000, 63999, 64000):
        assert H.audio_rows(n) == ref.encoder_output_length(-(-n // 160))
    assert H.audio_rows(64000) == 50
    assert H.chunk_lengths(80000) == [64000, 16000] and H.placeholder_rows(80000) == 50 + H.audio_rows(16000)
    assert (H.AUDIO_TOKEN, H.AUDIO_BOS, H.AUDIO_EOS) == (ref.audio_in_token_idx, ref.audio_bos_token_id, ref.audio_eos_token_id)
    assert {H.EOS, H.IM_END} == set(ref.stop_token_ids)
    assert H.llm_checkpoint_name("audio_tower.conv1.weight") is None
    assert H.llm_checkpoint_name("audio_decoder_proj.audio_lm_head.weight") is None
    assert H.llm_checkpoint_name(H.LM_HEAD) == H.LM_HEAD
    assert H.llm_checkpoint_name("model.layers.3.mlp.up_proj.weight") == "model.layers.3.mlp.up_proj.weight"


def test_served_rows_equal_placeholders():
    """The encoder node emits exactly the rows the prompt reserved, for whole, partial and very short chunks."""
    from types import SimpleNamespace
    from mstar_b200.models.higgs_audio import HiggsAudioModel, placeholder_rows
    m = HiggsAudioModel(small=True, skip_weight_loading=True)
    sub = m.get_submodule("audio_encoder", "cpu")
    for n in (300, 48000, 64000, 80000, 64001, 131000):
        wav = torch.randn(n) * 0.1
        ni = SimpleNamespace(tensor_inputs={"audio": [wav]}, kwargs={})
        rows = sub.forward("prefill_audio", None, ni)["audio_features"].shape[0]
        ids = m.process_prompt("transcribe", ["audio"], ["text"], {"audio": [wav]})["input_ids"][0]
        assert rows == placeholder_rows(n) == int((ids == 151672).sum()), (n, rows, placeholder_rows(n))


def test_model_loads_a_published_layout_directory(tmp_path):
    """A directory with the decoder (Qwen3 names, text head beside the audio heads), the tower, the projector and the
    speech-generation tensors the transcription model does not use."""
    from safetensors.torch import save_file
    from mstar_b200.models.higgs_audio import HiggsAudioModel, LM_HEAD
    m = HiggsAudioModel(model_dir=str(tmp_path), small=True)
    c, e = m.cfg, m.enc_cfg
    g = torch.Generator().manual_seed(3)
    r = lambda *s: torch.randn(s, generator=g) * 0.05  # noqa: E731
    H, D, Hq, Hkv, F = c.hidden_size, c.head_dim, c.num_heads, c.num_kv_heads, c.intermediate_size
    sd = {"model.embed_tokens.weight": r(c.vocab_size, H), "model.norm.weight": 1 + r(H), LM_HEAD: r(c.vocab_size, H),
          "audio_decoder_proj.audio_lm_head.weight": r(8, H), "audio_codebook_embeddings.weight": r(8, H)}
    for i in range(c.num_layers):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": r(Hq * D, H), p + "self_attn.k_proj.weight": r(Hkv * D, H),
                   p + "self_attn.v_proj.weight": r(Hkv * D, H), p + "self_attn.o_proj.weight": r(H, Hq * D),
                   p + "self_attn.q_norm.weight": 1 + r(D), p + "self_attn.k_norm.weight": 1 + r(D),
                   p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H),
                   p + "mlp.gate_proj.weight": r(F, H), p + "mlp.up_proj.weight": r(F, H), p + "mlp.down_proj.weight": r(H, F)})
    A, E = e.hidden_size, e.ffn_dim
    t = "audio_tower."
    sd.update({t + "conv1.weight": r(A, m.n_mels, 3), t + "conv1.bias": r(A), t + "conv2.weight": r(A, A, 3),
               t + "conv2.bias": r(A), t + "embed_positions.weight": r(1500, A), t + "layer_norm.weight": 1 + r(A),
               t + "layer_norm.bias": r(A)})
    for i in range(e.num_layers):
        p = f"{t}layers.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            sd[p + f"self_attn.{n}.weight"] = r(A, A)
            if n != "k_proj":
                sd[p + f"self_attn.{n}.bias"] = r(A)
        for n in ("self_attn_layer_norm", "final_layer_norm"):
            sd.update({p + n + ".weight": 1 + r(A), p + n + ".bias": r(A)})
        sd.update({p + "fc1.weight": r(E, A), p + "fc1.bias": r(E), p + "fc2.weight": r(A, E), p + "fc2.bias": r(A)})
    q = "audio_encoder_proj."
    sd.update({q + "temporal.weight": r(A, 1, 3), q + "temporal.bias": r(A), q + "linear1.weight": r(m.proj_mid, A),
               q + "linear1.bias": r(m.proj_mid), q + "linear2.weight": r(H, m.proj_mid), q + "linear2.bias": r(H)})
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    llm = m.get_submodule("LLM", "cpu")
    assert torch.equal(llm.lm.lm_head, sd[LM_HEAD]) and torch.equal(llm.lm.embed_tokens, sd["model.embed_tokens.weight"])
    assert not any(torch.isnan(p).any() for p in llm.lm.parameters())
    enc = m.get_submodule("audio_encoder", "cpu")
    assert torch.equal(enc.proj.w2, sd[q + "linear2.weight"]) and torch.equal(enc.enc.pos, sd[t + "embed_positions.weight"])
