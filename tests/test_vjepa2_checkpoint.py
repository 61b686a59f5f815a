"""V-JEPA 2 encoder and masked predictor against ``transformers.VJEPA2Model`` on shared weights (fp32, CPU), loaded
from the Hugging Face tensor names through the strict loaders."""
import pytest
import torch

from mstar_b200.engine.piecewise_graph import PiecewiseCudaGraphRunner
from mstar_b200.models import checkpoints as ck
from mstar_b200.models.encoders import EncoderConfig
from mstar_b200.models.vjepa2 import MaskedPredictor, VJepa2Encoder

transformers = pytest.importorskip("transformers")


def test_encoder_and_predictor_match_hugging_face_and_the_loaders_are_strict():
    torch.manual_seed(0)
    hc = transformers.VJEPA2Config(patch_size=4, crop_size=16, frames_per_clip=8, tubelet_size=2, hidden_size=48,
                                   in_chans=3, num_attention_heads=2, num_hidden_layers=2, mlp_ratio=2.0,
                                   pred_hidden_size=24, pred_num_attention_heads=2, pred_num_hidden_layers=2,
                                   pred_num_mask_tokens=3, pred_mlp_ratio=2.0, hidden_act="gelu")
    hf = transformers.VJEPA2Model(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.2)
        if "norm" in n and n.endswith("weight"):
            p.data.add_(1.0)
    sd = {k: v.clone() for k, v in hf.state_dict().items()}
    # head width 24: three rotary bands of 8 channels; head width 12 in the predictor: bands of 4
    c = EncoderConfig(48, 2, 2, 24, 96, norm="layernorm", act="gelu_erf", eps=hc.layer_norm_eps, dtype=torch.float32)
    pc = EncoderConfig(24, 2, 2, 12, 48, norm="layernorm", act="gelu_erf", eps=hc.layer_norm_eps, dtype=torch.float32)
    enc = VJepa2Encoder(c, patch=4, tubelet=2).init_random(0)
    pred = MaskedPredictor(48, pc, "cpu", num_mask_tokens=3).init_random(1)
    assert ck.load_vjepa2_encoder(enc, sd)["loaded"] == len(list(enc.parameters()))
    assert ck.load_vjepa2_predictor(pred, sd)["loaded"] == len(list(pred.parameters()))
    vid = torch.randn(3, 8, 16, 16)                          # [C, T, H, W]: 4 tubelet frames of 4 x 4 patches
    hf_in = vid.permute(1, 0, 2, 3)[None]                    # Hugging Face takes [B, T, C, H, W]
    with torch.no_grad():
        feats, lens, grids = enc([vid])
        want = hf(pixel_values_videos=hf_in, skip_predictor=True).last_hidden_state[0]
        assert lens == [64] and grids == [(4, 4, 4)]
        assert (feats - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item())
        perm = torch.randperm(64)
        tgt, ctx = perm[:20].sort().values, perm[20:].sort().values
        full = hf(pixel_values_videos=hf_in, context_mask=[ctx[None]], target_mask=[tgt[None]])
        got = pred(feats[ctx].contiguous(), ctx, tgt, PiecewiseCudaGraphRunner(False), (4, 4))
        want = full.predictor_output.last_hidden_state[0]
        assert got.shape == want.shape == (20, 48)
        assert (got - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item())
    for loader, module, mutate in (
            (ck.load_vjepa2_encoder, enc, lambda d: d.pop("encoder.layer.1.attention.key.bias")),
            (ck.load_vjepa2_encoder, enc, lambda d: d.update({"encoder.pos_embed": torch.zeros(4)})),
            (ck.load_vjepa2_predictor, pred, lambda d: d.update({"predictor.proj.weight": torch.zeros(48, 25)}))):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            loader(module, bad)
