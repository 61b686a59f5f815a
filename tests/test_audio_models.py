"""Speech models on CPU: Whisper-class decoder consistency (prefill + decode == longer prefill, cross-attention pool
slots), and the models through the serving stack with test-sized weights."""
import pytest
import torch

from mstar_b200.engine.cache_manager import BatchedCacheManager
from mstar_b200.engine.kv_store import KVCacheConfig


def test_whisper_decoder_incremental_equals_full_and_slots_are_independent():
    from mstar_b200.models.whisper import CrossAttnPool, WhisperDecoder
    dec = WhisperDecoder(vocab=300, hidden=64, layers=2, heads=4, ffn=128, dtype=torch.float32).init_random(1)
    for L in dec.layers:           # non-trivial biases
        L.qkv_b.data.normal_(0, 0.1)
        L.ckv_b.data.normal_(0, 0.1)
    pool = CrossAttnPool(2, 8, 40, 4, 16, torch.float32, "cpu")
    g = torch.Generator().manual_seed(0)
    feats = {"a": torch.randn(33, 64, generator=g), "b": torch.randn(17, 64, generator=g)}
    slots = {"a": 5, "b": 2}
    for r in feats:
        dec.project_cross(feats[r], pool, slots[r])
    ids = {"a": torch.randint(0, 300, (7,), generator=g), "b": torch.randint(0, 300, (4,), generator=g)}

    def fresh():
        kvc = KVCacheConfig(2, 4, 16, max_seq_len=64, max_num_pages=16, page_size=8, num_qo_heads=4, dtype=torch.float32)
        return BatchedCacheManager(kvc, "cpu", max_batch=4, max_tokens=64)
    # full prefill of both requests in one batch
    cm = fresh()
    ctx = cm.plan(["a", "b"], [7, 4], row_slots=[5, 2])
    full = dec(ctx, torch.cat([ids["a"], ids["b"]]), pool)
    # prefill without the last token, then one batched decode step
    cm = fresh()
    ctx = cm.plan(["a", "b"], [6, 3], row_slots=[5, 2])
    dec(ctx, torch.cat([ids["a"][:6], ids["b"][:3]]), pool)
    cm.advance_seq_lens(ctx)
    ctx = cm.plan(["b", "a"], [1, 1], row_slots=[2, 5])               # other order: slots, not rows, pick the audio
    step = dec(ctx, torch.stack([ids["b"][3], ids["a"][6]]), pool)
    assert (step[1] - full[0]).abs().max().item() < 1e-4
    assert (step[0] - full[1]).abs().max().item() < 1e-4
    # a request alone gives the same logits as inside the batch
    cm = fresh()
    solo = dec(cm.plan(["b"], [4], row_slots=[2]), ids["b"], pool)
    assert (solo[0] - full[1]).abs().max().item() < 1e-4


@pytest.fixture(scope="module")
def whisper_server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "whisper_large", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["audio_encoder"], "ranks": [0]}, {"node_names": ["decoder"], "ranks": [1]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def test_whisper_serving_two_requests(whisper_server):
    rids = [whisper_server.submit_request(None, output_modalities=["text"], model_kwargs=dict(max_tokens=5),
                                          tensors={"audio": [torch.randn(16000 * (i + 1)) * 0.1]}) for i in range(2)]
    for rid in rids:
        res = whisper_server.collect_results(rid, 120)
        assert "error" not in res and len(res["text"]) == 5


def test_higgs_audio_placeholders_are_replaced_by_encoder_frames():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "higgs_audio", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["audio_encoder", "LLM"], "ranks": [0]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        outs = []
        for wav in (torch.randn(16000 * 5) * 0.1, torch.randn(16000 * 5) * 0.3, None):
            rid = s.submit_request("transcribe", output_modalities=["text"], model_kwargs=dict(max_tokens=4),
                                   tensors={"audio": [wav]} if wav is not None else None)
            res = s.collect_results(rid, 120)
            assert "error" not in res and len(res["text"]) == 4, res
            outs.append(b"".join(c.data for c in res["text"]))
        # 5 s of audio = a 4 s chunk (50 rows) and a 1 s chunk (13 rows); different audio changes the continuation
        assert outs[0] != outs[1] or outs[0] != outs[2]
    finally:
        s.shutdown()


def test_qwen3_tts_streams_left_context_chunks():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "qwen3_tts", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["Talker"], "ranks": [0], "graph_walks": ["talker_prefill", "talker_decode"]},
                           {"node_names": ["Codec"], "ranks": [1], "graph_walks": ["codec_chunk"]}]}
    s = APIServer(cfg, in_process=True).start(120)
    try:
        rid = s.submit_request("hello world", output_modalities=["audio"], model_kwargs=dict(max_tokens=20, ignore_eos=True))
        res = s.collect_results(rid, 120)
        assert "error" not in res
        # 20 tokens = 1 prefill sample + 19 decode steps = 19 complete frames of 4 samples (hop 2*2), 2 bytes each:
        # chunks of 6 new frames (the context frames' samples are cut), then the flush
        sizes = [len(c.data) for c in res["audio"]]
        assert sum(sizes) == 19 * 4 * 2 and sizes[0] == 6 * 4 * 2, sizes
    finally:
        s.shutdown()


@pytest.fixture(scope="module")
def omni_server():
    from mstar_b200.api_server.server import APIServer
    cfg = {"model": "qwen3_omni", "model_kwargs": {"small": True}, "use_cuda_graphs": False,
           "node_groups": [{"node_names": ["audio_encoder", "vision_encoder", "Thinker"], "ranks": [0]},
                           {"node_names": ["Talker"], "ranks": [1]}, {"node_names": ["Code2Wav"], "ranks": [2]}]}
    s = APIServer(cfg, in_process=True).start(120)
    yield s
    s.shutdown()


def test_qwen3_omni_text_audio_image_in_text_out(omni_server):
    s = omni_server
    kw = dict(max_tokens=6, ignore_eos=True, temperature=0.0)
    a = s.collect_results(s.submit_request("describe", output_modalities=["text"], model_kwargs=kw), 120)
    b = s.collect_results(s.submit_request("describe", output_modalities=["text"], model_kwargs=kw,
                                           tensors={"audio": [torch.randn(8000) * 0.1], "image": [torch.rand(3, 16, 16)]}), 120)
    assert len(a["text"]) == 6 and len(b["text"]) == 6
    assert b"".join(c.data for c in a["text"]) != b"".join(c.data for c in b["text"])
    import time
    time.sleep(0.3)
    for w in s.deployment.workers:          # nothing of a text-only request stays behind on the speech workers
        assert len(w.tensors.store) == 0, (w.worker_id, len(w.tensors.store))


def test_qwen3_omni_speech_out_runs_three_partitions(omni_server):
    s = omni_server
    rid = s.submit_request("say hi", output_modalities=["text", "audio"],
                           model_kwargs=dict(max_tokens=5, ignore_eos=True, max_audio_tokens=15))
    res = s.collect_results(rid, 120)
    assert "error" not in res and len(res["text"]) == 5
    # 15 decode iterations -> 15 complete frames of 4 samples in three chunks; the causal transposed convolution at
    # the end of every chunk gives up its overhang of 2 samples
    assert sum(len(c.data) for c in res["audio"]) == (15 * 4 - 3 * 2) * 2


def test_mrope_positions_for_image_spans():
    from mstar_b200.models.qwen3_omni import IMAGE_TOKEN, mrope_positions
    ids = torch.tensor([5, 6, IMAGE_TOKEN, IMAGE_TOKEN, IMAGE_TOKEN, IMAGE_TOKEN, 7, 8])
    pos, delta = mrope_positions(ids, [(1, 2, 2)], IMAGE_TOKEN)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[:, 2:6].tolist() == [[2, 2, 2, 2], [2, 2, 3, 3], [2, 3, 2, 3]]
    assert pos[:, 6:].tolist() == [[4, 5]] * 3 and delta == 6 - 8


def test_qwen3_omni_talker_never_samples_control_codes():
    """The first code of a frame comes from the codebook or is the end-of-speech id: the other ids of the talker's
    vocabulary above the codebook are masked before sampling."""
    from mstar_b200.models.qwen3_omni import Qwen3OmniModel
    m = Qwen3OmniModel(small=True, skip_weight_loading=True)
    t = m.get_submodule("Talker", "cpu")
    V = m.k_cfg.vocab_size
    assert t.suppress is not None and int(t.suppress.sum()) == V - m.codebook - (1 if m.codec_eos >= m.codebook else 0)
    lg = torch.zeros(2, V)
    lg[:, V - 1] = 50.0                                   # a control id would win
    out = t._suppress(lg)
    assert m.codec_eos < m.codebook                       # the test-sized talker ends on a codebook id
    assert out.argmax(-1).max() < m.codebook and (out[:, m.codebook:] < -1e29).all()
    wide = t._suppress(torch.zeros(1, V + 8))             # a padded head keeps its pad columns
    assert wide.shape[-1] == V + 8 and (wide[0, V:] == 0).all()
