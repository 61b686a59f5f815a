"""Cosmos3 sound decoder: strict loading of the weight-normalised checkpoint layout and numerical parity with the
reference's decoder on the same checkpoint."""
import json
import os

import pytest
import torch

from mstar_b200.models.sound_decoder import SoundDecoder, load_sound_decoder, sound_decoder_config

from conftest import reference_module

CFG = dict(sampling_rate=480, dec_out_channels=2, vocoder_input_dim=8, dec_strides=[2, 3], dec_dim=8, dec_c_mults=[1, 2])


def _synthetic_checkpoint(dec: SoundDecoder, seed=0) -> dict:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for k, (kind, m) in dec.checkpoint_entries().items():
        if kind == "v":
            out[k] = torch.randn(m.weight.shape, generator=g) * 0.3
        elif kind == "g":
            shape = [m.weight.shape[0]] + [1] * (m.weight.dim() - 1)
            out[k] = torch.rand(shape, generator=g) + 0.5
        elif kind == "bias":
            out[k] = torch.randn(m.bias.shape, generator=g) * 0.1
        else:
            out[k] = torch.randn(1, m.a.shape[1], 1, generator=g) * 0.2
    out["encoder.conv1.bias"] = torch.zeros(3)          # a full auto-encoder file also carries an encoder
    return out


def test_strict_loading_and_geometry(tmp_path):
    dec = SoundDecoder(CFG)
    assert dec.hop_size == 6 and dec.latent_fps == 80.0 and dec.num_latent_frames(13) == 3
    ck = _synthetic_checkpoint(dec)
    d = tmp_path / "sound_tokenizer"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CFG))
    from safetensors.torch import save_file
    save_file(ck, str(d / "diffusion_pytorch_model.safetensors"))
    m = load_sound_decoder(str(tmp_path), dtype=torch.float32)
    wav = m.decode(torch.randn(2, 8, 5))
    assert wav.shape == (2, 2, 30) and wav.abs().max() <= 1.0
    for bad in ("missing", "unknown", "shape"):
        ck2 = dict(ck)
        if bad == "missing":
            ck2.pop("decoder.block.1.res_unit2.conv1.weight_g")
        elif bad == "unknown":
            ck2["decoder.block.7.snake1.alpha"] = torch.zeros(1)
        else:
            ck2["decoder.conv2.weight_v"] = torch.zeros(2, 8, 5)
        with pytest.raises((KeyError, ValueError)):
            SoundDecoder(CFG).load_checkpoint_tensors(ck2)


def test_parity_with_the_reference_decoder():
    ref = reference_module("mstar.model.cosmos3.components.sound_tokenizer")
    torch.manual_seed(0)
    rm = ref.Cosmos3SoundTokenizer(dict(CFG)).eval()
    with torch.no_grad():
        for n, p in rm.named_parameters():
            p.copy_(torch.randn_like(p) * (0.2 if ("alpha" in n or "beta" in n) else 0.3))
            if n.endswith("weight_g"):
                p.abs_().add_(0.5)
    ours = SoundDecoder(CFG)
    ours.load_checkpoint_tensors({k: v.detach().clone() for k, v in rm.state_dict().items()})
    z = torch.randn(2, 8, 7)
    want = rm.decode(z.clone())
    got = ours.decode(z)
    assert got.shape == want.shape == (2, 2, 42)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), (got - want).abs().max()
    # the tanh-normalised latent variant
    cfg2 = dict(CFG, normalization_type="tanh")
    rm2 = ref.Cosmos3SoundTokenizer(cfg2).eval()
    rm2.load_state_dict(rm.state_dict())
    o2 = SoundDecoder(cfg2)
    o2.load_checkpoint_tensors({k: v.detach().clone() for k, v in rm.state_dict().items()})
    assert torch.allclose(o2.decode(z), rm2.decode(z.clone()), atol=2e-5, rtol=1e-4)
