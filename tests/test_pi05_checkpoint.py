"""Pi0.5 policy from a checkpoint in the published (lerobot) key layout: strictness of the loader, the prefix tower
against Hugging Face Gemma, and the served action chunk against a plain PyTorch fp32 restatement of the whole policy
(Hugging Face SigLIP + Gemma for the prefix, the adaptive-norm action expert written out below)."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from safetensors.torch import save_file

from mstar_b200.models import checkpoints as ck
from mstar_b200.models.pi05 import Pi05Model, Pi05Policy

PALI = "paligemma_with_expert.paligemma.model."
EXPERT = "paligemma_with_expert.gemma_expert.model."
KW = dict(vocab=1024, hidden=64, layers=2, heads=4, kv_heads=1, head_dim=16, ffn=128, a_hidden=32, a_ffn=64)


def _policy(seed):
    m = Pi05Policy(action_dim=32, dtype=torch.float32, device="cpu", **KW).init_random(seed)
    g = torch.Generator().manual_seed(seed + 100)
    for n, p in m.named_parameters():
        if p.dim() == 1:
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
        elif "mod" in n:                                  # visible scale / shift / gate modulation
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.2)
    return m


def _hf_gemma():
    from transformers import GemmaConfig, GemmaModel
    hc = GemmaConfig(vocab_size=KW["vocab"], hidden_size=KW["hidden"], intermediate_size=KW["ffn"],
                     num_hidden_layers=KW["layers"], num_attention_heads=KW["heads"], num_key_value_heads=KW["kv_heads"],
                     head_dim=KW["head_dim"], hidden_act="gelu_pytorch_tanh", rms_norm_eps=1e-6, rope_theta=10000.0,
                     attention_bias=False, pad_token_id=0, bos_token_id=2, eos_token_id=1)
    torch.manual_seed(1)
    hf = GemmaModel(hc).float().eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.12)
    return hf


def _with_hf_prefix(sd, hf):
    for k, v in hf.state_dict().items():
        if k == "embed_tokens.weight":
            sd["paligemma_with_expert.paligemma.lm_head.weight"] = v.clone()
        else:
            sd[PALI + "language_model." + k] = v.clone()
    return sd


def test_pi05_loader_round_trips_and_is_strict():
    a = _policy(0)
    sd = ck.pi05_checkpoint_keys(a)
    sd["paligemma_with_expert.gemma_expert.lm_head.weight"] = torch.zeros(4, 4)       # unused by the policy: ignored
    sd[PALI + "vision_tower.vision_model.post_layernorm.weight"] = torch.zeros(4)     # another node's: ignored here
    b = _policy(7)
    assert ck.load_pi05_policy(b, sd)["loaded"] == len(list(a.parameters()))
    assert all(torch.equal(x, y) for x, y in zip(a.parameters(), b.parameters()))
    for mutate in (lambda d: d.pop(EXPERT + "layers.1.post_attention_layernorm.dense.bias"),
                   lambda d: d.update({EXPERT + "layers.0.input_layernorm.weight": torch.zeros(32)}),
                   lambda d: d.update({"action_out_proj.weight": torch.zeros(32, 33)}),
                   lambda d: d.pop("paligemma_with_expert.paligemma.lm_head.weight")):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_pi05_policy(_policy(1), bad)


def test_pi05_prefix_tower_matches_hugging_face_gemma_with_a_bidirectional_mask():
    from mstar_b200.ops import attention as attn_ops
    hf, m = _hf_gemma(), _policy(0)
    ck.load_pi05_policy(m, _with_hf_prefix(ck.pi05_checkpoint_keys(m), hf))
    n = 11
    x = torch.randn(n, KW["hidden"])
    with torch.no_grad():
        want = hf(inputs_embeds=x[None], attention_mask=torch.zeros(1, 1, n, n),
                  position_ids=torch.arange(n)[None]).last_hidden_state[0]
        plan = attn_ops.dense_plan([n], [n], KW["heads"] // KW["kv_heads"], "cpu", causal=False)
        pos, h = torch.arange(n, dtype=torch.int32), x
        for li in range(KW["layers"]):
            h = m.und.layer(li, h, pos, lambda i, q, k, v: attn_ops.attention(q, plan, k=k, v=v))
        got = m.und.final(h)
    assert (got - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item())


# ---------------------------------------------------------------- the whole policy, restated in plain PyTorch
def _rms(x):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)


def _ada(x, cond, w, b):
    scale, shift, gate = (cond @ w.T + b).chunk(3, dim=-1)
    return _rms(x) * (1 + scale) + shift, gate


def _rot(x, pos, D):
    """x: [n, heads, D]; rotate-half rotary embedding at integer positions ``pos``."""
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    return x * cos + torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1) * sin


def _expert_velocity(sd, x, t, prefix_kv, pos0):
    A, nh, nkv, D = KW["a_hidden"], KW["heads"], KW["kv_heads"], KW["head_dim"]
    n = x.shape[0]
    h = x @ sd["action_in_proj.weight"].T + sd["action_in_proj.bias"]
    frac = torch.linspace(0, 1, A // 2, dtype=torch.float64)
    period = 4e-3 * (4.0 / 4e-3) ** frac
    ang = t * 2 * math.pi / period
    e = torch.cat([ang.sin(), ang.cos()]).float()[None]
    c = F.silu(e @ sd["time_mlp_in.weight"].T + sd["time_mlp_in.bias"])
    c = F.silu(c @ sd["time_mlp_out.weight"].T + sd["time_mlp_out.bias"])
    pos = torch.arange(n) + pos0
    for li in range(KW["layers"]):
        p = f"{EXPERT}layers.{li}."
        hn, gate = _ada(h, c, sd[p + "input_layernorm.dense.weight"], sd[p + "input_layernorm.dense.bias"])
        q = _rot((hn @ sd[p + "self_attn.q_proj.weight"].T).reshape(n, nh, D), pos, D)
        k = _rot((hn @ sd[p + "self_attn.k_proj.weight"].T).reshape(n, nkv, D), pos, D)
        v = (hn @ sd[p + "self_attn.v_proj.weight"].T).reshape(n, nkv, D)
        K = torch.cat([prefix_kv[li][0], k]).repeat_interleave(nh // nkv, 1)        # [S + n, nh, D]
        V = torch.cat([prefix_kv[li][1], v]).repeat_interleave(nh // nkv, 1)
        w = torch.softmax(torch.einsum("qhd,khd->hqk", q, K) / math.sqrt(D), dim=-1)
        o = torch.einsum("hqk,khd->qhd", w, V).reshape(n, nh * D)
        h = h + gate * (o @ sd[p + "self_attn.o_proj.weight"].T)
        hn, gate = _ada(h, c, sd[p + "post_attention_layernorm.dense.weight"], sd[p + "post_attention_layernorm.dense.bias"])
        y = F.gelu(hn @ sd[p + "mlp.gate_proj.weight"].T, approximate="tanh") * (hn @ sd[p + "mlp.up_proj.weight"].T)
        h = h + gate * (y @ sd[p + "mlp.down_proj.weight"].T)
    hn, _ = _ada(h, c, sd[EXPERT + "norm.dense.weight"], sd[EXPERT + "norm.dense.bias"])
    return hn @ sd["action_out_proj.weight"].T + sd["action_out_proj.bias"]


def test_pi05_served_actions_match_a_plain_pytorch_policy_on_a_published_layout_checkpoint(tmp_path):
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from mstar_b200.api_server.server import APIServer
    hf = _hf_gemma()
    sd = _with_hf_prefix(ck.pi05_checkpoint_keys(_policy(3)), hf)
    torch.manual_seed(2)
    vis = SiglipVisionModel(SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                               num_attention_heads=2, num_channels=3, image_size=16, patch_size=4,
                                               vision_use_head=False)).float().eval()
    for p in vis.parameters():
        torch.nn.init.normal_(p, std=0.1)
    proj_w, proj_b = torch.randn(KW["hidden"], 32) * 0.2, torch.randn(KW["hidden"]) * 0.1
    for k, v in vis.state_dict().items():
        sd[PALI + "vision_tower." + k] = v.clone()
    sd[PALI + "multi_modal_projector.linear.weight"], sd[PALI + "multi_modal_projector.linear.bias"] = proj_w, proj_b
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))

    imgs = [torch.rand(3, 16, 16), torch.rand(3, 16, 16)]
    prompt, state, seed, steps, horizon = "pick up the cup", [0.1, -0.5], 3, 10, 8
    cfg = {"model": "pi05", "model_dir": str(tmp_path), "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["vit_encoder"], "ranks": [0]}, {"node_names": ["LLM"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        rid = s.submit_request(prompt, output_modalities=["action"], model_kwargs=dict(seed=seed, state=state),
                               tensors={"image": imgs})
        res = s.collect_results(rid, 120)
        assert "error" not in res, res
        got = torch.from_numpy(np.frombuffer(res["action"][0].data, dtype=np.float32).reshape(horizon, 32).copy())
    finally:
        s.shutdown()

    H = KW["hidden"]
    ids = Pi05Model(small=True).process_prompt(prompt, ["text"], ["action"], {"image": imgs}, state=state)["input_ids"][0]
    with torch.no_grad():
        feats = vis(pixel_values=torch.stack(imgs) * 2 - 1).last_hidden_state            # [2, 16, 32]
        img_tok = (feats @ proj_w.T + proj_b).reshape(-1, H) * math.sqrt(H)
        txt_tok = hf.embed_tokens.weight[ids] * H
        x = torch.cat([img_tok, txt_tok])
        S = x.shape[0]
        out = hf(inputs_embeds=x[None], attention_mask=torch.zeros(1, 1, S, S), position_ids=torch.arange(S)[None],
                 use_cache=True)
        kv = [(out.past_key_values.layers[li].keys[0].transpose(0, 1), out.past_key_values.layers[li].values[0].transpose(0, 1))
              for li in range(KW["layers"])]
        a = torch.randn((horizon, 32), generator=torch.Generator().manual_seed(seed))
        for i in range(steps):
            a = a - _expert_velocity(sd, a, 1.0 - i / steps, kv, S) / steps
    assert torch.isfinite(got).all()
    assert (got - a).abs().max().item() < 2e-3 * max(1.0, a.abs().max().item()), (got - a).abs().max().item()


def test_pi05_prompt_follows_the_published_format_when_the_checkpoint_has_a_tokenizer():
    seen = []

    class Tok:
        def __call__(self, text, add_special_tokens=True):
            seen.append((text, add_special_tokens))
            return type("Enc", (), {"input_ids": list(range(2, 2 + 300))})()
    m = Pi05Model(small=True)
    m._hf_tokenizer = Tok()
    out = m.process_prompt("Pick_up the\nCup ", ["text"], ["action"], {"image": [torch.rand(3, 16, 16)]},
                           robot_state=[-1.0, 0.0, 1.0, 2.0])
    assert seen == [("task: pick up the cup, state: 0 128 255 255;\naction:", True)]
    assert out["input_ids"][0].numel() == Pi05Model.MAX_LANG_TOKENS
