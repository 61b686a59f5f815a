"""DiT family on CPU (fp32 oracles of the kernels): the AdaLN block stack against an independent plain-torch
restatement, prefix/fresh attention merge against one attention over the concatenated keys, sampler sanity, VAE
shapes, and the Wan2.2-class model through the serving stack."""
import math

import pytest
import torch
import torch.nn.functional as F

from mstar_b200.models.dit import AdaLNDiT, DiTConfig, grid_positions, patchify, sinusoidal_embedding, unpatchify
from mstar_b200.models.schedulers import FlowEulerSchedule, FlowUniPC
from mstar_b200.models.vae import ConvVAE, tiny_vae_config
from mstar_b200.ops import attention as attn_ops


def _rms(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def _rope_complex(x, pos, axes, theta):
    """x: [S, heads, D]; pos [3, S]; consecutive pairs rotate; bands of the head dim belong to (t, h, w)."""
    S, nh, D = x.shape
    xc = torch.view_as_complex(x.double().reshape(S, nh, D // 2, 2))
    freqs = []
    for a, d in enumerate(axes):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        freqs.append(torch.polar(torch.ones(S, d // 2, dtype=torch.float64), pos[a].double()[:, None] * inv[None]))
    out = torch.view_as_real(xc * torch.cat(freqs, dim=1)[:, None]).reshape(S, nh, D)
    return out.float()


def _ref_forward(m: AdaLNDiT, latents, timesteps, text_embs):
    c = m.cfg
    H, nh, D = c.hidden_size, c.num_heads, c.head_dim
    outs = []
    for b in range(latents.shape[0]):
        tok, grid = patchify(latents[b], c.patch_size)
        S = tok.shape[0]
        x = F.linear(tok, m.patch_w, m.patch_b)
        e = sinusoidal_embedding(timesteps[b].reshape(-1), c.freq_dim)
        e = F.linear(F.silu(F.linear(e, m.time1_w, m.time1_b)), m.time2_w, m.time2_b)          # [n, H]
        e6 = F.linear(F.silu(e), m.tproj_w, m.tproj_b).reshape(-1, 6, H)
        rep = S // e6.shape[0]
        ctx = F.linear(F.gelu(F.linear(text_embs[b], m.text1_w, m.text1_b), approximate="tanh"), m.text2_w, m.text2_b)
        pos = grid_positions(*grid, "cpu")
        for blk in m.blocks:
            mod = (blk.modulation[None] + e6).repeat_interleave(rep, 0)                           # [S, 6, H]
            h = F.layer_norm(x, (H,), eps=c.eps) * (1 + mod[:, 1]) + mod[:, 0]
            qkv = F.linear(h, blk.qkv_w, blk.qkv_b)
            q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
            q, k = _rms(q, blk.norm_q, c.eps), _rms(k, blk.norm_k, c.eps)
            q = _rope_complex(q.reshape(S, nh, D), pos, c.axes(), c.rope_theta)
            k = _rope_complex(k.reshape(S, nh, D), pos, c.axes(), c.rope_theta)
            a = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.reshape(S, nh, D).transpose(0, 1))
            x = x + mod[:, 2] * F.linear(a.transpose(0, 1).reshape(S, H), blk.o_w, blk.o_b)
            h = F.layer_norm(x, (H,), blk.norm3_w, blk.norm3_b, eps=c.eps)
            q = _rms(F.linear(h, blk.cq_w, blk.cq_b), blk.cnorm_q, c.eps).reshape(S, nh, D)
            kv = F.linear(ctx, blk.ckv_w, blk.ckv_b)
            kk = _rms(kv[:, :H], blk.cnorm_k, c.eps).reshape(-1, nh, D)
            vv = kv[:, H:].reshape(-1, nh, D)
            a = F.scaled_dot_product_attention(q.transpose(0, 1), kk.transpose(0, 1), vv.transpose(0, 1))
            x = x + F.linear(a.transpose(0, 1).reshape(S, H), blk.co_w, blk.co_b)
            h = F.layer_norm(x, (H,), eps=c.eps) * (1 + mod[:, 4]) + mod[:, 3]
            h = F.linear(F.gelu(F.linear(h, blk.ffn1_w, blk.ffn1_b), approximate="tanh"), blk.ffn2_w, blk.ffn2_b)
            x = x + mod[:, 5] * h
        hm = (m.head_mod[None] + e[:, None]).repeat_interleave(rep, 0)
        h = F.layer_norm(x, (H,), eps=c.eps) * (1 + hm[:, 1]) + hm[:, 0]
        outs.append(unpatchify(F.linear(h, m.head_w, m.head_b), grid, c.patch_size, c.out_channels))
    return torch.stack(outs)


@pytest.mark.parametrize("per_frame_t", [False, True])
def test_adaln_dit_matches_plain_torch(per_frame_t):
    cfg = DiTConfig(hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_dim=128, in_channels=4,
                    out_channels=4, text_dim=32, text_len=8, dtype=torch.float32, rope_axes=(4, 6, 6))
    m = AdaLNDiT(cfg).init_random(3)
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, 4, 3, 8, 8, generator=g)
    texts = [torch.randn(8, 32, generator=g), torch.randn(5, 32, generator=g)]
    ts = torch.tensor([[700.0, 700.0, 700.0], [0.0, 300.0, 300.0]]) if per_frame_t else torch.tensor([700.0, 300.0])
    kv = m.encode_context(torch.cat(texts))
    out = m(lat, ts, kv, [8, 5])
    ref = _ref_forward(m, lat, ts.reshape(2, -1), texts)
    assert out.shape == lat.shape
    assert (out - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())


def test_patchify_roundtrip():
    x = torch.randn(4, 3, 8, 6)
    tok, grid = patchify(x, (1, 2, 2))
    assert grid == (3, 4, 3) and tok.shape == (36, 16)
    # unpatchify expects channel-fastest tokens: permute the patch vector accordingly
    t2 = tok.reshape(36, 4, 1, 2, 2).permute(0, 2, 3, 4, 1).reshape(36, 16)
    assert torch.equal(unpatchify(t2, grid, (1, 2, 2), 4), x)


def test_prefix_and_fresh_attention_merge_equals_joint_attention():
    g = torch.Generator().manual_seed(1)
    T, Hq, Hkv, D, Lp = 12, 4, 2, 16, 9
    q = torch.randn(T, Hq, D, generator=g)
    kp, vp = torch.randn(Lp, Hkv, D, generator=g), torch.randn(Lp, Hkv, D, generator=g)
    kf, vf = torch.randn(T, Hkv, D, generator=g), torch.randn(T, Hkv, D, generator=g)
    G = Hq // Hkv
    o1, l1 = attn_ops.attention(q, attn_ops.dense_plan([T], [Lp], G, "cpu"), k=kp, v=vp, lse=True)
    o2, l2 = attn_ops.attention(q, attn_ops.dense_plan([T], [T], G, "cpu"), k=kf, v=vf, lse=True)
    merged = attn_ops.attn_merge(o1, l1, o2, l2)
    joint = attn_ops.attention(q, attn_ops.dense_plan([T], [Lp + T], G, "cpu"), k=torch.cat([kp, kf]), v=torch.cat([vp, vf]))
    assert (merged - joint).abs().max().item() < 1e-5
    # an empty prefix contributes nothing
    e = attn_ops.attn_merge(torch.zeros_like(o2), torch.full_like(l2, -math.inf), o2, l2)
    assert torch.allclose(e, o2)


def test_unipc_is_exact_on_a_straight_flow_and_agrees_with_euler_in_the_limit():
    g = torch.Generator().manual_seed(0)
    data, noise = torch.randn(3, 5, generator=g), torch.randn(3, 5, generator=g)
    s = FlowUniPC(6, shift=5.0)
    x = noise.clone()
    for _ in range(6):
        x = s.step(noise - data, x)
    assert (x - data).abs().max().item() < 1e-5

    def model(x, sig):
        return (x - torch.tanh(x)) / max(sig, 1e-3)
    N = 400
    s, e = FlowUniPC(N, shift=3.0), FlowEulerSchedule(N, 3.0)
    x, y = noise.clone(), noise.clone()
    for i in range(N):
        x = s.step(model(x, s.sigmas[i]), x)
        y = e.step(y, model(y, e.sigmas[i]), i)
    assert (x - y).abs().max().item() < 5e-3


def test_vae_shapes_2d_and_causal_3d():
    v2 = ConvVAE(tiny_vae_config(2)).eval()
    x = torch.rand(1, 3, 16, 16) * 2 - 1
    z = v2.encode(x)
    assert z.shape == (1, 4, 8, 8) and v2.decode(z).shape == x.shape
    v3 = ConvVAE(tiny_vae_config(3)).eval()
    x = torch.rand(1, 3, 5, 16, 16) * 2 - 1
    z = v3.encode(x)
    assert z.shape == (1, 4, 3, 8, 8) and v3.decode(z).shape == x.shape
    # causal in time: the first latent frame depends on the first pixel frame only
    x2 = x.clone()
    x2[:, :, 1:] = 0
    assert torch.allclose(v3.encode(x2)[:, :, 0], z[:, :, 0], atol=1e-5)


@pytest.fixture(scope="module")
def wan_server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "wan22", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["text_encoder", "vae_encoder"], "ranks": [0]},
                           {"node_names": ["dit", "vae_decoder"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def test_wan22_text_to_video_and_image_to_video(wan_server):
    kw = dict(num_steps=3, height=16, width=16, num_frames=5, seed=7)
    a = wan_server.collect_results(wan_server.submit_request("a red fox", output_modalities=["video"], model_kwargs=kw), 120)
    b = wan_server.collect_results(wan_server.submit_request("a red fox", output_modalities=["video"], model_kwargs=kw), 120)
    assert a["video"][0].data[:4] == b"RIFF" and a["video"][0].data == b["video"][0].data          # seeded: reproducible
    c = wan_server.collect_results(wan_server.submit_request(
        "a red fox", output_modalities=["video"], model_kwargs=kw, tensors={"image": [torch.rand(3, 16, 16) * 2 - 1]}), 120)
    assert c["video"][0].data[:4] == b"RIFF" and c["video"][0].data != a["video"][0].data


@pytest.fixture(scope="module")
def cosmos_server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "cosmos3", "model_kwargs": {"small": True, "page_size": 16, "max_num_pages": 64},
           "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["dit"], "ranks": [0]},
                           {"node_names": ["vae_encoder", "vae_decoder", "audio_decoder"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


@pytest.mark.parametrize("outs,with_image", [(["image"], False), (["video"], False), (["video", "audio"], False),
                                              (["action"], False), (["video"], True)])
def test_cosmos3_walks(cosmos_server, outs, with_image):
    kw = dict(num_steps=3, height=16, width=16, num_frames=5, negative_prompt="blurry", seed=3)
    rid = cosmos_server.submit_request("a robot arm", output_modalities=outs, model_kwargs=kw,
                                       tensors={"image": [torch.rand(3, 16, 16) * 2 - 1]} if with_image else None)
    res = cosmos_server.collect_results(rid, 120)
    assert set(res) == set(outs), res.keys()
    if "image" in res:
        assert res["image"][0].data[:4] == b"\x89PNG"
    if "action" in res:
        assert len(res["action"][0].data) == 16 * 32 * 4
    # the request's pages went back to the pool
    eng = cosmos_server.deployment.workers[0].engines.engine_for("dit")
    import time
    for _ in range(100):
        if eng.cache.alloc.pages_of(rid) == 0:
            break
        time.sleep(0.02)
    assert eng.cache.alloc.pages_of(rid) == 0


def test_cosmos3_tp2_sp2_matches_single_rank_on_gloo():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", "4", os.path.join(root, "tests", "mp_cosmos_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES="", MSTAR_TEST_BACKEND="gloo"), cwd=root)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
