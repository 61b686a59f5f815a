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
