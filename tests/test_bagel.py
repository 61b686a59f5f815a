"""BAGEL-class mixture-of-transformers on CPU: the per-expert row split of the packed prefill, and the model through
the serving stack (understanding, text-to-image, editing, and packed vs. CFG-parallel guidance)."""
import pytest
import torch

from mstar_b200.engine.cache_manager import BatchedCacheManager
from mstar_b200.engine.kv_store import KVCacheConfig
from mstar_b200.models.bagel import BagelMoT
from mstar_b200.models.decoder import DecoderConfig


def _cm():
    kvc = KVCacheConfig(2, 2, 16, max_seq_len=64, max_num_pages=16, page_size=8, num_qo_heads=4, dtype=torch.float32)
    return BatchedCacheManager(kvc, "cpu", max_batch=4, max_tokens=64)


def test_mixed_expert_prefill_equals_plain_decoder_when_experts_share_weights():
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                        vocab_size=300, qkv_bias=True, qk_norm=True, dtype=torch.float32)
    m = BagelMoT(cfg, 16).init_random(0)
    for lu, lg in zip(m.und.layers, m.gen.layers):     # generation expert := understanding expert
        lu.self_attn.qkv_bias.data.normal_(0, 0.05)
        lg.input_norm.data.copy_(lu.input_layernorm.data.normal_(1, 0.1))
        lg.post_norm.data.copy_(lu.post_attention_layernorm.data.normal_(1, 0.1))
        lg.qkv_proj.data.copy_(lu.self_attn.qkv_proj.data)
        lg.qkv_bias.data.copy_(lu.self_attn.qkv_bias.data)
        lg.q_norm.data.copy_(lu.self_attn.q_norm.data.normal_(1, 0.1))
        lg.k_norm.data.copy_(lu.self_attn.k_norm.data.normal_(1, 0.1))
        lg.o_proj.data.copy_(lu.self_attn.o_proj.data)
        lg.gate_up_proj.data.copy_(lu.mlp.gate_up_proj.data)
        lg.down_proj.data.copy_(lu.mlp.down_proj.data)
    m.gen.final_norm.data.copy_(m.und.norm.data.normal_(1, 0.1))
    g = torch.Generator().manual_seed(0)
    x = torch.randn(11, 64, generator=g)
    cm = _cm()
    ref = m.und.forward_hidden(x.clone(), cm.plan(["a"], [11]))
    for mask in (torch.zeros(11, dtype=torch.bool), torch.arange(11) % 3 == 1, torch.ones(11, dtype=torch.bool)):
        cm = _cm()
        out = m.forward_mixed(x.clone(), mask, cm.plan(["a"], [11]))
        assert (out - ref).abs().max().item() < 1e-4


def test_experts_differ_when_weights_differ():
    cfg = DecoderConfig(hidden_size=64, num_layers=1, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                        vocab_size=300, dtype=torch.float32)
    m = BagelMoT(cfg, 16).init_random(0)
    x = torch.randn(6, 64, generator=torch.Generator().manual_seed(1))
    a = m.forward_mixed(x.clone(), torch.zeros(6, dtype=torch.bool), _cm().plan(["a"], [6]))
    b = m.forward_mixed(x.clone(), torch.tensor([0, 0, 1, 1, 0, 0], dtype=torch.bool), _cm().plan(["a"], [6]))
    assert (a[:2] - b[:2]).abs().max().item() < 1e-5          # causal: rows before the first generation row agree
    assert (a[2:] - b[2:]).abs().max().item() > 1e-3


def test_packed_prefill_with_an_image_span_equals_text_image_text_passes():
    """One packed pass (causal rows + the span's rows redone without a mask up to the span's end) gives the hidden
    states of the reference's procedure: causal text pass, bidirectional image pass, causal text pass, each
    extending the cache; the rows of a span share one rotary position."""
    from mstar_b200.models.bagel import IMG_PLACEHOLDER, VAE_PLACEHOLDER, VISION_END, VISION_START, image_span_positions
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                        vocab_size=300, qkv_bias=True, qk_norm=True, dtype=torch.float32)
    m = BagelMoT(cfg, 16).init_random(0)
    ids = [5, 6, 7, VISION_START] + [VAE_PLACEHOLDER] * 4 + [VISION_END, 8, 9]
    pos, spans = image_span_positions(ids)
    assert pos.tolist() == [0, 1, 2, 3, 3, 3, 3, 3, 3, 4, 5] and spans == [(3, 9)]
    assert image_span_positions([VISION_START, IMG_PLACEHOLDER, VISION_END, 4])[0].tolist() == [0, 0, 0, 1]
    x = torch.randn(len(ids), 64, generator=torch.Generator().manual_seed(2))
    is_gen = torch.tensor([t == VAE_PLACEHOLDER for t in ids])
    cm = _cm()
    ctx = cm.plan(["a"], [len(ids)], custom_positions=pos[None].to(torch.int32), group=2)
    one = m.forward_mixed(x.clone(), is_gen, ctx, spans=cm.span_plan(ctx, [(0, 3, 9)], group=2))
    causal_only = m.forward_mixed(x.clone(), is_gen, _cm().plan(["a"], [len(ids)], custom_positions=pos[None].to(torch.int32)))
    cm2, parts = _cm(), []
    for a, b, causal in ((0, 3, True), (3, 9, False), (9, 11, True)):
        c = cm2.plan(["a"], [b - a], causal=causal, custom_positions=pos[None, a:b].to(torch.int32), group=2)
        parts.append(m.forward_mixed(x[a:b].clone(), is_gen[a:b], c))
        cm2.advance_seq_lens(c)
    want = torch.cat(parts)
    assert (one - want).abs().max().item() < 1e-4
    assert (causal_only[:3] - want[:3]).abs().max().item() < 1e-5       # rows before the span never see it
    assert (causal_only[3:8] - want[3:8]).abs().max().item() > 1e-3     # rows inside the span see its later rows
    with pytest.raises(ValueError):
        cm.span_plan(ctx, [(0, 9, 12)])


@pytest.fixture(scope="module")
def server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "bagel", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["vit_encoder", "vae_encoder", "LLM", "vae_decoder"], "ranks": [0]},
                           {"node_names": ["LLM_cfg_text"], "ranks": [1]},
                           {"node_names": ["LLM_cfg_img", "combine_cfg"], "ranks": [2]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def _run(s, outs, tensors=None, **kw):
    mk = dict(max_tokens=5, ignore_eos=True, num_steps=3, height=16, width=16, seed=1, **kw)
    res = s.collect_results(s.submit_request("a cat", output_modalities=outs, model_kwargs=mk, tensors=tensors), 120)
    assert "error" not in res, res
    return res


def test_understanding_with_and_without_image(server):
    a = _run(server, ["text"])
    b = _run(server, ["text"], {"image": [torch.rand(3, 16, 16)]})
    assert len(a["text"]) == 5 and len(b["text"]) == 5


def test_text_to_image_packed_equals_cfg_parallel(server):
    a = _run(server, ["image"])
    b = _run(server, ["image"], cfg_parallel=True)
    assert set(a) == {"image"} and a["image"][0].data[:4] == b"\x89PNG"
    import io

    import numpy as np
    from PIL import Image
    pa, pb = (np.asarray(Image.open(io.BytesIO(r["image"][0].data)), dtype=np.int32) for r in (a, b))
    assert pa.shape == pb.shape and np.abs(pa - pb).max() <= 2          # same picture up to rounding
    c = _run(server, ["image"], cfg_text_scale=1.0)
    pc = np.asarray(Image.open(io.BytesIO(c["image"][0].data)), dtype=np.int32)
    assert np.abs(pa - pc).max() > 2                                    # guidance does change the picture


def test_image_editing_uses_three_contexts(server):
    img = torch.rand(3, 16, 16)
    a = _run(server, ["image"], {"image": [img]}, cfg_img_scale=1.5)
    b = _run(server, ["image"], {"image": [img]}, cfg_img_scale=1.0)
    assert a["image"][0].data != b["image"][0].data


def test_packed_deployment_without_the_guidance_parallel_nodes():
    """The guidance-parallel nodes are optional: a one-group deployment serves the packed walks and refuses, by name,
    a request that asks for the parallel ones."""
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "bagel", "model_kwargs": {"small": True},
           "node_groups": [{"node_names": ["vit_encoder", "vae_encoder", "LLM", "vae_decoder"], "ranks": [0]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        kw = dict(height=32, width=32, num_steps=3, cfg_text_scale=4.0, seed=0)
        rid = s.submit_request("a cat", output_modalities=["image"], model_kwargs=kw)
        assert s.collect_results(rid, 120)["image"][0].data[:4] == b"\x89PNG"
        rid = s.submit_request("a cat", output_modalities=["image"], model_kwargs=dict(kw, cfg_parallel=True))
        res = s.collect_results(rid, 120)
        assert "error" in res and b"LLM_cfg" in res["error"][0].data
    finally:
        s.shutdown()


def test_a_deployment_whose_process_dies_at_start_up_fails_fast():
    from mstar_b200.api_server.server import APIServer
    bad = {"model": "bagel", "model_kwargs": {"small": True}, "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
    import time
    t0 = time.time()
    try:
        APIServer(bad, in_process=False).start(300)
        raise AssertionError("start-up should have failed: most nodes are not placed")
    except (RuntimeError, ValueError):
        pass
    assert time.time() - t0 < 120


def test_per_walk_placement_gives_the_same_tokens_and_images_as_one_gpu():
    """The prompt passes on one rank, decoding and image generation on others (the LLM node placed per walk): the
    request's KV pages of every guidance context move at the walk switch, the node runs only where its walk is
    placed, and understanding, text-to-image and editing give what the single-rank placement gives — repeatedly."""
    import hashlib
    import yaml
    import torch
    from mstar_b200.api_server.server import APIServer

    def run(path):
        cfg = yaml.safe_load(open(path))
        cfg.update(model_kwargs={"small": True}, use_cuda_graphs=False)
        torch.manual_seed(0)                      # the test-sized autoencoder takes torch's default initialisation
        s = APIServer(cfg, in_process=True).start(120)
        out = []
        try:
            mk = dict(max_tokens=5, ignore_eos=True, num_steps=3, height=16, width=16, seed=1, temperature=0.0)
            img = torch.rand(3, 16, 16, generator=torch.Generator().manual_seed(3))
            for _ in range(2):
                for prompt, outs, tens in (("a cat", ["text"], {"image": [img]}), ("a cat", ["image"], None),
                                           ("make it blue", ["image"], {"image": [img]})):
                    r = s.collect_results(s.submit_request(prompt, output_modalities=outs, model_kwargs=mk, tensors=tens), 120)
                    assert "error" not in r, r
                    out.append(hashlib.md5(b"".join(c.data for c in r[outs[0]])).hexdigest())
            assert out[:3] == out[3:]
            import time
            for w in s.deployment.workers:       # every page goes back, on every rank (the teardown message follows the result)
                eng = w.engines.engine_for("LLM")
                for _ in range(100):
                    if eng.cache.alloc.num_free_pages == eng.cache.alloc.total_pages:
                        break
                    time.sleep(0.02)
                assert eng.cache.alloc.num_free_pages == eng.cache.alloc.total_pages
        finally:
            s.shutdown()
        return out
    single = run("configs/bagel_single_gpu.yaml")
    assert run("configs/bagel_pd_disaggregated.yaml") == single
    assert run("configs/bagel_img_disaggregated.yaml") == single
