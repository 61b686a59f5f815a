"""Orpheus-class TTS through the serving stack on CPU with a test-sized backbone: LLM partition streams audio
tokens into the codec partition in sliding windows (28 / 7); audio chunks come back as PCM16."""
import pytest

from mstar_b200.api_server.server import APIServer

CFG = {"model": "orpheus", "model_kwargs": {"small": True, "page_size": 16, "max_num_pages": 256},
       "use_cuda_graphs": False,
       "node_groups": [{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                       {"node_names": ["snac_decoder"], "ranks": [1], "graph_walks": ["snac_chunk"]}]}


@pytest.fixture(scope="module")
def server():
    s = APIServer(CFG, in_process=True).start(120)
    yield s
    s.shutdown()


def test_tts_streams_audio_chunks(server):
    n_tokens = 7 * 9      # 9 frames
    rid = server.submit_request("hello there", output_modalities=["audio"],
                                model_kwargs=dict(max_tokens=n_tokens, ignore_eos=True, voice="leo"))
    chunks = list(server.iter_result_chunks(rid, 300))
    assert chunks and all(c.modality == "audio" for c in chunks), [c.modality for c in chunks][:5]
    # windows: the first full window appears after 28 tokens, then one per frame, then the flush
    sizes = [len(c.data) // 2 for c in chunks]
    assert sizes.count(2048) >= 5
    assert sum(sizes) >= 2048 * 6
    assert server.deployment.conductor.stats["completed"] >= 1


def test_two_requests_share_the_codec_worker(server):
    rids = [server.submit_request(f"req {i}", output_modalities=["audio"],
                                  model_kwargs=dict(max_tokens=35, ignore_eos=True)) for i in range(2)]
    for rid in rids:
        res = server.collect_results(rid, 300)
        assert "error" not in res and len(res["audio"]) >= 2


def test_prefill_decode_disaggregation_moves_the_kv_pages():
    """Prefill on worker 0, decode on worker 1 (separate page pools): tokens equal the colocated run's."""
    base = {"model": "tiny", "use_cuda_graphs": False}
    pd = dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill"]},
                                 {"node_names": ["LLM"], "ranks": [1], "graph_walks": ["decode"]}])
    co = dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0]}])
    outs = []
    for cfg in (co, pd):
        s = APIServer(cfg, in_process=True).start(120)
        try:
            rid = s.submit_request("the quick brown fox jumps over the lazy dog", output_modalities=["text"],
                                   model_kwargs=dict(max_tokens=12, ignore_eos=True, temperature=0.7, top_p=0.9,
                                                     repetition_penalty=1.2, seed=5))
            res = s.collect_results(rid, 300)
            assert "error" not in res, res
            outs.append(b"".join(c.data for c in res["text"]))
            if cfg is pd:
                pre, dec = (w.engines.engine_for("LLM") for w in s.deployment.workers[:2])
                assert dec.graph_hits == 0 and pre.cache.alloc is not dec.cache.alloc
        finally:
            s.shutdown()
    assert len(outs[0]) > 0 and outs[0] == outs[1]


def test_colocated_partitions_share_one_worker():
    """LLM and codec partitions on the same worker: the stream goes to the codec partition's request state."""
    cfg = dict(CFG, node_groups=[{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                                 {"node_names": ["snac_decoder"], "ranks": [0], "graph_walks": ["snac_chunk"]}])
    s = APIServer(cfg, in_process=True).start(120)
    try:
        rid = s.submit_request("hello there", output_modalities=["audio"], model_kwargs=dict(max_tokens=63, ignore_eos=True))
        sizes = [len(c.data) for c in s.iter_result_chunks(rid, 300)]
        assert sizes.count(4096) >= 5 and sum(sizes) >= 4096 * 8, sizes
    finally:
        s.shutdown()


def test_middle_frame_decode_equals_the_slice_of_the_full_window():
    """A streaming window of four frames yields its second frame; decoding only the positions that frame depends on
    (receptive field of the residual stacks and transposed convolutions, stage by stage) gives the same samples as
    slicing them out of the full decode — also at the signal's edges and for odd upsampling rates."""
    import torch
    from mstar_b200.models.codec import SnacDecoder
    torch.manual_seed(0)
    for kw in (dict(latent_dim=64, channels=64, rates=(8, 8, 4, 2)), dict(latent_dim=32, channels=32, rates=(3, 5, 2))):
        d = SnacDecoder(noise=False, **kw).eval()
        for p in d.parameters():
            p.data.normal_(0, 0.04)
        codes = [torch.randint(0, 4096, (2, 4)), torch.randint(0, 4096, (2, 8)), torch.randint(0, 4096, (2, 16))]
        with torch.no_grad():
            full = d(codes)
            hop = d.hop
            assert full.shape[1] == 16 * hop and full.abs().max().item() > 1e-3
            for lo, hi in ((4 * hop, 8 * hop), (0, 4 * hop), (12 * hop, 16 * hop), (5, 77)):
                part = d(codes, keep=(lo, hi))
                assert part.shape == (2, hi - lo)
                assert (part - full[:, lo:hi]).abs().max().item() < 1e-6
        # at the codec's own rates the finest stage sees about a quarter of the window
        need = [(max(0, 4 * hop - 3), 8 * hop + 3)]
        lens = [16]
        for b in d.blocks:
            lens.append(lens[-1] * b.up[1].stride[0])
        ra, rb, _, _ = d.blocks[-1].input_range(*need[0], lens[-2])
        if hop == 512:
            assert (rb - ra) < 0.3 * lens[-1]


def test_snac_decoder_loads_the_published_layout_and_matches_the_reference_module():
    """The reference's own ``SNAC`` (the published 24 kHz architecture at test width: depthwise convolutions, noise
    blocks, weight normalisation) and ``SnacDecoder`` loaded from its state dict decode the same codes to the same
    waveform, with the noise drawn from the same generator state; the loader refuses what does not fit."""
    import inspect
    import pytest
    import torch
    from conftest import reference_module
    snac_mod = reference_module("mstar.model.orpheus.components.snac")
    from mstar_b200.models import checkpoints as ck
    from mstar_b200.models.codec import SnacDecoder
    cfg = dict(sampling_rate=24000, encoder_dim=8, encoder_rates=[2, 4, 8, 8], latent_dim=48, decoder_dim=64,
               decoder_rates=[8, 8, 4, 2], attn_window_size=None, codebook_size=4096, codebook_dim=8,
               vq_strides=[4, 2, 1], noise=True, depthwise=True)
    ok = set(inspect.signature(snac_mod.SNAC.__init__).parameters)
    torch.manual_seed(0)
    ref = snac_mod.SNAC(**{k: v for k, v in cfg.items() if k in ok}).eval()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if "alpha" in n:
                p.uniform_(0.5, 1.5)
            elif n.endswith("bias"):
                p.normal_(0, 0.05)
    sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    ours = SnacDecoder(latent_dim=48, channels=64, rates=(8, 8, 4, 2)).eval()
    assert ck.load_snac_decoder(ours, sd)["loaded"] == len(list(ours.parameters()))
    codes = [torch.randint(0, 4096, (2, 4)), torch.randint(0, 4096, (2, 8)), torch.randint(0, 4096, (2, 16))]
    with torch.no_grad():
        torch.manual_seed(7)
        want = ref.decode(codes)[:, 0]
        torch.manual_seed(7)
        got = ours(codes)
        assert got.shape == want.shape == (2, 16 * 512)
        assert (got - want).abs().max().item() < 1e-5 and want.abs().max().item() > 1e-3
    for mutate in (lambda d: d.pop("decoder.model.3.block.2.linear.parametrizations.weight.original1"),
                   lambda d: d.update({"decoder.model.9.extra": torch.zeros(1)}),
                   lambda d: d.update({"quantizer.quantizers.1.codebook.weight": torch.zeros(4096, 9)})):
        bad = dict(sd)
        mutate(bad)
        with pytest.raises(ck.CheckpointMismatch):
            ck.load_snac_decoder(SnacDecoder(latent_dim=48, channels=64, rates=(8, 8, 4, 2)), bad)
