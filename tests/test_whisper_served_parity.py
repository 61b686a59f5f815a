"""Whisper served from a checkpoint in the Hugging Face layout: the greedy tokens that the serving stack emits (audio
encoder, cross-attention pool, paged self-attention decode loop) equal a plain greedy loop over
``transformers.WhisperForConditionalGeneration`` with the same weights and the same log-mel input."""
import pytest
import torch
from safetensors.torch import save_file

transformers = pytest.importorskip("transformers")


def test_served_whisper_tokens_equal_hugging_face_greedy_decoding(tmp_path):
    from mstar_b200.api_server.server import APIServer
    from mstar_b200.models.encoders import log_mel_spectrogram
    from mstar_b200.models.whisper import LANG_EN, NO_TS, SOT, TRANSCRIBE
    cfg = transformers.WhisperConfig(vocab_size=51866, num_mel_bins=16, d_model=64, encoder_layers=2, decoder_layers=2,
                                     encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=128,
                                     decoder_ffn_dim=128, max_source_positions=200, max_target_positions=448,
                                     dropout=0.0, attention_dropout=0.0, activation_dropout=0.0, pad_token_id=0,
                                     bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)
    torch.manual_seed(3)
    hf = transformers.WhisperForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "encoder.embed_positions" not in n:
                p.copy_(torch.randn_like(p) * (0.12 if p.dim() > 1 else 0.05) + (1.0 if "layer_norm.weight" in n else 0.0))
    sd = {k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()}
    save_file(sd, str(tmp_path / "model.safetensors"))
    wav = torch.randn(64000, generator=torch.Generator().manual_seed(5)) * 0.1          # 4 s: one full window here
    n_new = 8
    srv = APIServer({"model": "whisper_large", "model_dir": str(tmp_path), "model_kwargs": {"small": True},
                     "use_cuda_graphs": False, "node_groups": [{"node_names": ["audio_encoder", "decoder"], "ranks": [0]}]},
                    in_process=True).start(120)
    try:
        res = srv.collect_results(srv.submit_request("transcribe", output_modalities=["text"],
                                                     model_kwargs=dict(max_tokens=n_new, ignore_eos=True, temperature=0.0),
                                                     tensors={"audio": [wav]}), 120)
        assert "error" not in res, res
        got = [int(t) for t in b"".join(c.data for c in res["text"]).decode().split()]
    finally:
        srv.shutdown()
    mel = log_mel_spectrogram(wav, n_mels=16)
    assert mel.shape == (16, 400)
    ids = torch.tensor([[SOT, LANG_EN, TRANSCRIBE, NO_TS]])
    with torch.no_grad():
        enc = hf.model.encoder(mel[None]).last_hidden_state
        want = []
        for _ in range(n_new):
            logits = hf(encoder_outputs=(enc,), decoder_input_ids=ids).logits[0, -1]
            want.append(int(logits.argmax()))
            ids = torch.cat([ids, torch.tensor([[want[-1]]])], dim=1)
    assert got == want
