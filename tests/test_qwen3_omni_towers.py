"""Qwen3-Omni towers against the Hugging Face modules on shared weights (fp32, CPU): the audio tower, the vision
tower with its deepstack taps, and the thinker's decoder (mixture of experts, q/k norms, interleaved 3-axis rotary
positions, deepstack features added to the first layers' outputs), each loaded through the strict checkpoint loaders
from the published tensor names."""
import pytest
import torch
from safetensors.torch import save_file

from mstar_b200.models import checkpoints as ck
from mstar_b200.models.encoders import EncoderConfig
from mstar_b200.models.qwen3_omni_encoders import OmniAudioEncoder, OmniVisionEncoder, audio_output_length

hf_omni = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
hf_cfg = pytest.importorskip("transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe")


def _hf_audio(n_window_infer):
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=16, encoder_layers=2, encoder_attention_heads=2,
                                               encoder_ffn_dim=64, d_model=32, max_source_positions=64, n_window=50,
                                               output_dim=24, n_window_infer=n_window_infer, downsample_hidden_size=8)
    hf = hf_omni.Qwen3OmniMoeAudioEncoder(hc).float().eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.2)
    c = EncoderConfig(32, 2, 2, 16, 64, norm="layernorm", act="gelu_erf", eps=1e-5, dtype=torch.float32)
    ours = OmniAudioEncoder(c, n_mels=16, conv_channels=8, out_dim=24, n_window=50, n_window_infer=n_window_infer,
                            max_positions=64).init_random(0)
    sd = {"thinker.audio_tower." + k: v.clone() for k, v in hf.state_dict().items()}
    return hf, ours, sd


def test_audio_tower_matches_hugging_face_and_the_loader_is_strict():
    hf, ours, sd = _hf_audio(800)                  # one attention window covers the clip
    assert ck.load_qwen3_omni_audio(ours, sd)["loaded"] == len(list(ours.parameters()))
    mel, mel2 = torch.randn(16, 437), torch.randn(16, 230)
    with torch.no_grad():
        want = hf(mel, feature_lens=torch.tensor([437])).last_hidden_state
        got, lens = ours([mel])
        assert lens == [57] == [audio_output_length(437)] and got.shape == want.shape
        assert (got - want).abs().max().item() < 1e-4
        both, lens2 = ours([mel, mel2])            # clips are independent of their batch neighbours
        assert lens2 == [57, audio_output_length(230)]
        assert (both[:57] - want).abs().max().item() < 1e-4
    for mutate in (lambda d: d.pop("thinker.audio_tower.conv_out.weight"),
                   lambda d: d.update({"thinker.audio_tower.layers.0.extra.weight": torch.zeros(2)}),
                   lambda d: d.update({"thinker.audio_tower.proj2.weight": torch.zeros(24, 31)})):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_qwen3_omni_audio(ours, bad)


def test_audio_tower_attention_stays_inside_its_windows():
    """Windows of ``n_window_infer`` input frames (26 rows here): against the Hugging Face layers run with the
    block-diagonal mask that their variable-length attention path stands for."""
    hf, ours, sd = _hf_audio(200)
    ck.load_qwen3_omni_audio(ours, sd)
    mel = torch.randn(16, 437)
    with torch.no_grad():
        got, _ = ours([mel])
        x = torch.stack([torch.nn.functional.pad(p, (0, 100 - p.shape[1])) for p in mel.split(100, dim=1)])[:, None]
        for conv in (hf.conv2d1, hf.conv2d2, hf.conv2d3):
            x = torch.nn.functional.gelu(conv(x))
        n, ch, f, t = x.shape
        x = hf.conv_out(x.permute(0, 3, 1, 2).reshape(n, t, ch * f)) + hf.positional_embedding.positional_embedding[:t]
        h = torch.cat([x[i, :r] for i, r in enumerate([13, 13, 13, 13, 5])])
        cu = torch.tensor([0, 26, 52, 57], dtype=torch.int32)
        mask = hf._prepare_attention_mask(h, cu)
        for layer in hf.layers:
            h = layer(h, cu, attention_mask=mask)[0]
        want = hf.proj2(hf.act(hf.proj1(hf.ln_post(h))))
    assert (got - want).abs().max().item() < 1e-4


def test_vision_tower_and_deepstack_taps_match_hugging_face():
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeVisionEncoderConfig(depth=3, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4,
                                                spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=24,
                                                num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
    hf = hf_omni.Qwen3OmniMoeVisionEncoder(hc).float().eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.2)
    c = EncoderConfig(32, 3, 2, 16, 64, norm="layernorm", act="gelu", eps=1e-6, dtype=torch.float32)
    ours = OmniVisionEncoder(c, patch=4, temporal_patch=2, merge=2, pos_grid=6, out_dim=24, deepstack=(0, 2)).init_random(0)
    sd = {"thinker.visual." + k: v.clone() for k, v in hf.state_dict().items()}
    assert ck.load_qwen3_omni_vision(ours, sd)["loaded"] == len(list(ours.parameters()))
    img, clip = torch.randn(3, 16, 24), torch.randn(3, 4, 8, 8)      # 4 x 6 patches; two frames of 2 x 2 patches
    with torch.no_grad():
        got, deep, lens, grids = ours([img, clip])
        px = torch.cat([ours.patches(img)[0], ours.patches(clip)[0]])
        out = hf(px, grid_thw=torch.tensor([[1, 4, 6], [2, 2, 2]]))
    assert lens == [6, 2] and grids == [(1, 4, 6), (2, 2, 2)]
    assert (got - out.pooler_output).abs().max().item() < 1e-4
    assert len(deep) == 2 and all((d - w).abs().max().item() < 1e-4 for d, w in zip(deep, out.deepstack_features))
    # the pixel layout handed to the Hugging Face tower: a merge block's patches adjacent, (C, t, y, x) inside a patch
    first = ours.patches(img)[0][1].reshape(3, 2, 4, 4)
    assert torch.equal(first[:, 0], img[:, 0:4, 4:8]) and torch.equal(first[:, 1], img[:, 0:4, 4:8])
    bad = dict(sd)
    bad.pop("thinker.visual.merger_list.1.ln_q.bias")
    with pytest.raises(ck.CheckpointMismatch):
        ck.load_qwen3_omni_vision(ours, bad)


def test_thinker_decoder_matches_hugging_face_with_interleaved_mrope_and_deepstack(tmp_path):
    from mstar_b200.engine.cache_manager import BatchedCacheManager
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.models.decoder import DecoderConfig, DecoderLM
    from mstar_b200.models.loader import load_decoder_from_hf
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeTextConfig(
        vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, num_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=32, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], attention_bias=False,
        pad_token_id=0, rope_parameters={"rope_type": "default", "rope_theta": 1e6, "mrope_section": [2, 3, 3],
                                         "mrope_interleaved": True})
    hf = hf_omni.Qwen3OmniMoeThinkerTextModel(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.1)
        if "norm" in n:
            p.data.add_(1.0)
    sd = {}                                 # the published checkpoint stores every expert's projections separately
    for k, v in hf.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, dim=0)
                base = "thinker.model." + k[:-len("gate_up_proj")] + f"{e}."
                sd[base + "gate_proj.weight"], sd[base + "up_proj.weight"] = g.clone(), u.clone()
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                sd["thinker.model." + k[:-len("down_proj")] + f"{e}.down_proj.weight"] = v[e].clone()
        else:
            sd["thinker.model." + k] = v.clone()
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    cfg = DecoderConfig(hidden_size=64, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=200, rope_theta=1e6, qk_norm=True, mrope_sections=[2, 3, 3], mrope_interleaved=True,
                        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True,
                        has_lm_head=False, dtype=torch.float32)
    lm = DecoderLM(cfg)
    assert not load_decoder_from_hf(lm, str(tmp_path), prefix="thinker.model.")["incomplete"]
    T = 12
    ids = torch.randint(0, 200, (T,))
    pos = torch.tensor([[0, 1, 2, 3, 3, 3, 3, 5, 6, 7, 8, 9], [0, 1, 2, 3, 3, 4, 4, 5, 6, 7, 8, 9],
                        [0, 1, 2, 3, 4, 3, 4, 5, 6, 7, 8, 9]])           # a 2 x 2 image span at rows 3..6
    rows = torch.tensor([3, 4, 5, 6])
    deep = [torch.randn(4, 64) * 0.5 for _ in range(2)]
    mask = torch.zeros(1, T, dtype=torch.bool)
    mask[0, rows] = True
    kvc = KVCacheConfig(3, 2, 16, max_seq_len=64, max_num_pages=8, page_size=16, num_qo_heads=4, dtype=torch.float32)
    with torch.no_grad():
        want = hf(input_ids=ids[None], position_ids=pos[:, None], visual_pos_masks=mask,
                  deepstack_visual_embeds=deep).last_hidden_state[0]
        plain = hf(input_ids=ids[None], position_ids=pos[:, None]).last_hidden_state[0]
        outs = []
        for ds in ((rows, deep), None):
            cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64, n_pos_axes=3)
            cm.add_request("r")
            ctx = cm.plan(["r"], [T], custom_positions=pos.to(torch.int32), group=2)
            outs.append(lm.forward_hidden(lm.embed(ids), ctx, deepstack=ds))
    assert (outs[0] - want).abs().max().item() < 1e-4
    assert (outs[1] - plain).abs().max().item() < 1e-4
    assert (want - plain).abs().max().item() > 1e-2


def test_code2wav_matches_hugging_face_and_chunks_continue_each_other():
    from mstar_b200.models.code2wav import OmniCode2Wav
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeCode2WavConfig(codebook_size=32, hidden_size=32, num_attention_heads=2, num_key_value_heads=2,
                                           sliding_window=5, intermediate_size=48, num_hidden_layers=2, num_quantizers=4,
                                           upsample_rates=[3, 2], upsampling_ratios=[2, 2], decoder_dim=16,
                                           max_position_embeddings=256)
    hf = hf_omni.Qwen3OmniMoeCode2Wav(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.08)
        if "norm" in n and n.endswith("weight"):
            p.data.add_(1.0)
    ours = OmniCode2Wav(n_codebooks=4, codebook_size=32, hidden=32, layers=2, heads=2, head_dim=16, ffn=48, window=5,
                        upsampling_ratios=(2, 2), upsample_rates=(3, 2), decoder_dim=16).init_random(0)
    sd = {"code2wav." + k: v.clone() for k, v in hf.state_dict().items()}
    assert ck.load_qwen3_omni_code2wav(ours, sd)["loaded"] == len(list(ours.parameters()))
    assert ours.pre.inv_freq.dtype == torch.float32
    codes = torch.randint(0, 32, (2, 4, 13))                  # 13 frames: longer than the attention window of 5
    with torch.no_grad():
        want, got = hf(codes)[:, 0], ours(codes)
        assert want.abs().max().item() < 1.0                  # not saturated: the comparison sees the whole stack
        assert got.shape == want.shape and (got - want).abs().max().item() < 1e-5
        whole = hf.chunked_decode(codes, chunk_size=6, left_context_size=2)[:, 0]
        parts, start = [], 0
        while start < 13:
            ctx = 2 if start - 2 > 0 else start
            parts.append(ours(codes[..., start - ctx:min(start + 6, 13)])[:, ctx * ours.hop:])
            start += 6
        assert (torch.cat(parts, dim=-1) - whole).abs().max().item() < 1e-5
    for mutate in (lambda d: d.pop("code2wav.decoder.2.block.3.act2.beta"),
                   lambda d: d.update({"code2wav.pre_transformer.layers.0.self_attn.q_norm.weight": torch.ones(16)}),
                   lambda d: d.update({"code2wav.upsample.1.1.gamma": torch.zeros(31)})):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_qwen3_omni_code2wav(ours, bad)


def test_talker_backbone_with_its_gated_shared_expert_matches_hugging_face(tmp_path):
    """``talker.model.*`` (routed experts plus a sigmoid-gated shared expert, token table under ``codec_embedding``)
    loaded by the strict decoder loader against ``Qwen3OmniMoeTalkerModel``."""
    from mstar_b200.engine.cache_manager import BatchedCacheManager
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.models.decoder import DecoderConfig, DecoderLM
    from mstar_b200.models.loader import load_decoder_from_hf
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeTalkerTextConfig(
        vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, num_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=32, shared_expert_intermediate_size=48, norm_topk_prob=True, decoder_sparse_step=1,
        mlp_only_layers=[], attention_bias=False, pad_token_id=0,
        rope_parameters={"rope_type": "default", "rope_theta": 1e6, "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    hf = hf_omni.Qwen3OmniMoeTalkerModel(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.1)
        if "norm" in n:
            p.data.add_(1.0)
    sd = {"talker.codec_head.weight": torch.randn(96, 64) * 0.1}
    for k, v in hf.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, dim=0)
                base = "talker.model." + k[:-len("gate_up_proj")] + f"{e}."
                sd[base + "gate_proj.weight"], sd[base + "up_proj.weight"] = g.clone(), u.clone()
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                sd["talker.model." + k[:-len("down_proj")] + f"{e}.down_proj.weight"] = v[e].clone()
        else:
            sd["talker.model." + k] = v.clone()
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=96, rope_theta=1e6, qk_norm=True, num_experts=4, num_experts_per_tok=2,
                        moe_intermediate_size=32, shared_expert_intermediate_size=48, norm_topk_prob=True,
                        dtype=torch.float32)
    lm = DecoderLM(cfg)
    info = load_decoder_from_hf(lm, str(tmp_path), prefix="talker.model.", head_name="talker.codec_head.weight",
                                embed_name="codec_embedding.weight")
    assert not info["missing"] and torch.equal(lm.embed_tokens, sd["talker.model.codec_embedding.weight"])
    assert torch.equal(lm.lm_head, sd["talker.codec_head.weight"])
    T = 9
    ids = torch.randint(0, 96, (T,))
    kvc = KVCacheConfig(2, 2, 16, max_seq_len=64, max_num_pages=8, page_size=16, num_qo_heads=4, dtype=torch.float32)
    with torch.no_grad():
        x = hf.codec_embedding(ids)
        want = hf(inputs_embeds=x[None], position_ids=torch.arange(T)[None, None].expand(3, 1, T)).last_hidden_state[0]
        cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64)
        cm.add_request("r")
        got = lm.forward_hidden(lm.embed(ids), cm.plan(["r"], [T], group=2))
    assert (got - want).abs().max().item() < 1e-4


def test_code_predictor_gives_hugging_face_greedy_codes():
    """``talker.code_predictor.*`` loaded into ``CodePredictor``: the residual codes of a frame, decoded greedily from
    the talker's hidden state and first code, equal the Hugging Face module's cached generation (prefill over
    [hidden, first-code embedding], then one step per code layer through its own embedding table and head)."""
    from mstar_b200.models.decoder import DecoderConfig
    from mstar_b200.models.talker import CodePredictor
    torch.manual_seed(0)
    hc = hf_cfg.Qwen3OmniMoeTalkerCodePredictorConfig(
        vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
        num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, num_code_groups=4, attention_bias=False,
        max_position_embeddings=64, rope_parameters={"rope_type": "default", "rope_theta": 1e6}, pad_token_id=0)
    hf = hf_omni.Qwen3OmniMoeTalkerCodePredictorModelForConditionalGeneration(hc).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.2)
        if "norm" in n:
            p.data.add_(1.0)
    talker_table = torch.randn(96, 32) * 0.3                 # the talker's own token table embeds the first code
    sd = {"talker.code_predictor." + k: v.clone() for k, v in hf.state_dict().items()}
    sd["talker.model.codec_embedding.weight"] = talker_table
    cfg = DecoderConfig(hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, intermediate_size=48,
                        vocab_size=8, qk_norm=True, rope_theta=1e6, rms_eps=1e-6, dtype=torch.float32)
    pred = CodePredictor(cfg, 32, 3, 64, "cpu").init_random(0)
    assert ck.load_qwen3_omni_code_predictor(pred, sd)["loaded"] == len(list(pred.parameters()))
    hidden, code0 = torch.randn(3, 32), torch.randint(0, 64, (3,))
    with torch.no_grad():
        got = pred(hidden, code0, None, None)
        out = hf(inputs_embeds=torch.stack([hidden, talker_table[code0]], dim=1), use_cache=True)
        codes = [code0]
        for g in range(3):
            codes.append(out.logits[:, -1].argmax(-1))
            if g < 2:
                out = hf(input_ids=codes[-1][:, None], past_key_values=out.past_key_values, use_cache=True,
                         generation_steps=g + 1)
    assert torch.equal(got, torch.stack(codes, dim=1))
    bad = dict(sd)
    bad.pop("talker.code_predictor.lm_head.2.weight")
    with pytest.raises(ck.CheckpointMismatch):
        ck.load_qwen3_omni_code_predictor(pred, bad)
    with pytest.raises(ck.CheckpointMismatch):               # a predictor narrower than the talker has no such layout
        ck.load_qwen3_omni_code_predictor(CodePredictor(cfg, 48, 3, 64, "cpu").init_random(0), sd)
