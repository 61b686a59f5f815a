"""Decode bursts: several decode steps per node execution (device-side token feedback) give exactly the tokens of
single-step decoding, stop at EOS inside a burst, respect the token budget, and feed stream buffers item by item.
Runs on CPU with the engine's eager stand-in for captured graphs."""
import os

import pytest

from mstar_b200.api_server.server import APIServer


def _tokens(burst, graphs, eos_ids=(), **mk):
    os.environ["MSTAR_EMULATE_GRAPHS"] = "1" if graphs else ""
    os.environ["MSTAR_DECODE_BURST"] = str(burst)
    try:
        cfg = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 256, "eos_ids": list(eos_ids)},
               "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
        s = APIServer(cfg, in_process=True).start(60)
        try:
            outs = []
            rids = [s.submit_request(p, output_modalities=["text"], model_kwargs=dict(mk)) for p in ("1 2 3", "7 8 9 10 11")]
            for r in rids:
                res = s.collect_results(r, 120)
                assert "error" not in res, res
                outs.append(b"".join(c.data for c in res["text"]).decode().split())
            eng = s.deployment.workers[0].engines.engine_for("LLM")
            _tokens.spec = dict(s.deployment.workers[0].spec_stats)
            return outs, eng.graph_hits
        finally:
            s.shutdown()
    finally:
        os.environ.pop("MSTAR_EMULATE_GRAPHS", None)
        os.environ.pop("MSTAR_DECODE_BURST", None)


def test_speculative_bursts_give_the_same_tokens_and_drop_rows_past_a_stop():
    """While burst N is on the device the worker queues burst N+1 for the same requests (its inputs are the ids that
    N leaves in the engine's static buffer). Tokens must equal the unspeculated run; a request that meets its stop
    token in burst N has its row of burst N+1 dropped."""
    # Greedy here: with two requests the batch composition of the first steps depends on timing (one request may
    # decode alone for a burst), and fp32 results of different batch sizes differ in their last bits. That is enough
    # to flip a SAMPLED token of this nearly flat toy distribution, but not its argmax.
    kw = dict(max_tokens=41, ignore_eos=True, temperature=0.0)
    os.environ["MSTAR_SPECULATE"] = "0"
    try:
        ref, _ = _tokens(4, True, **kw)
        assert _tokens.spec["launched"] == 0
    finally:
        os.environ.pop("MSTAR_SPECULATE", None)
    got, _ = _tokens(4, True, **kw)
    assert _tokens.spec["launched"] > 0, _tokens.spec
    assert got == ref and all(len(t) == 41 for t in got)
    # stop tokens: greedy run, then declare a mid-sequence token of the first request the stop token
    plain, _ = _tokens(1, True, max_tokens=30, ignore_eos=True, temperature=0.0)
    stop = int(plain[0][9])
    first = plain[0].index(str(stop))
    out, _ = _tokens(3, True, eos_ids=[stop], max_tokens=30, temperature=0.0)
    assert out[0] == plain[0][:first + 1]
    os.environ["MSTAR_SPECULATE"] = "0"
    try:
        unspec, _ = _tokens(3, True, eos_ids=[stop], max_tokens=30, temperature=0.0)
    finally:
        os.environ.pop("MSTAR_SPECULATE", None)
    assert out == unspec


def test_burst_decoding_equals_single_step_decoding():
    kw = dict(max_tokens=23, ignore_eos=True, temperature=0.8, top_p=0.9, repetition_penalty=1.1, seed=11)
    ref, hits0 = _tokens(1, False, **kw)
    one, hits1 = _tokens(1, True, **kw)
    five, hits5 = _tokens(5, True, **kw)
    assert hits0 == 0 and hits1 > 0 and hits5 > 0
    assert ref == one == five
    assert all(len(t) == 23 for t in five)          # 1 prefill token + 22 decode tokens: budget respected in bursts


def test_burst_is_cut_at_the_stop_token():
    # greedy decoding of the tiny model: declare a token that appears mid-sequence the stop token
    ref, _ = _tokens(1, True, max_tokens=16, ignore_eos=True, temperature=0.0)
    stop = int(ref[0][6])
    first = ref[0].index(str(stop))
    out, _ = _tokens(4, True, eos_ids=[stop], max_tokens=16, temperature=0.0)
    assert out[0] == ref[0][:first + 1]
    one, _ = _tokens(1, True, eos_ids=[stop], max_tokens=16, temperature=0.0)
    assert one == out


def test_tts_stream_with_frame_sized_bursts():
    """Orpheus-class model: bursts of 7 tokens (one audio frame) reach the codec's sliding window item by item."""
    os.environ["MSTAR_EMULATE_GRAPHS"] = "1"
    try:
        cfg = {"model": "orpheus", "model_kwargs": {"small": True, "page_size": 16, "max_num_pages": 256},
               "node_groups": [{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill", "decode"]},
                               {"node_names": ["snac_decoder"], "ranks": [0], "graph_walks": ["snac_chunk"]}]}
        s = APIServer(cfg, in_process=True).start(120)
        try:
            rid = s.submit_request("hello there", output_modalities=["audio"], model_kwargs=dict(max_tokens=63, ignore_eos=True))
            sizes = [len(c.data) for c in s.iter_result_chunks(rid, 300)]
            eng = s.deployment.workers[0].engines.engine_for("LLM")
            assert eng.decode_burst == 7 and eng.graph_hits >= 56
            # 63 tokens = 9 frames: six full windows (one frame of audio each) and the flush of the last three
            assert sizes.count(4096) == 6 and sum(sizes) == 4096 * 9, sizes
        finally:
            s.shutdown()
    finally:
        os.environ.pop("MSTAR_EMULATE_GRAPHS", None)


def _run_requests(prompts, **mk):
    """Tokens of each prompt when all of them are submitted together (one decode batch, padded to its bucket)."""
    os.environ["MSTAR_EMULATE_GRAPHS"] = "1"
    os.environ["MSTAR_DECODE_BURST"] = "1"
    try:
        cfg = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 256},
               "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
        s = APIServer(cfg, in_process=True).start(60)
        try:
            rids = [s.submit_request(p, output_modalities=["text"], request_id=f"pad-{p.replace(' ', '_')}",
                                     model_kwargs=dict(mk)) for p in prompts]
            outs = {}
            for p, r in zip(prompts, rids):
                res = s.collect_results(r, 120)
                assert "error" not in res, res
                outs[p] = b"".join(c.data for c in res["text"]).decode().split()
            return outs
        finally:
            s.shutdown()
    finally:
        os.environ.pop("MSTAR_EMULATE_GRAPHS", None)
        os.environ.pop("MSTAR_DECODE_BURST", None)


def test_padding_rows_do_not_disturb_a_seeded_penalised_request():
    """Three requests decode in the bucket of four: the padding row samples with the sampler's reserved slot, so a
    request's repetition-penalty mask and draw counter are the same as when it runs alone in the bucket of one."""
    kw = dict(max_tokens=20, ignore_eos=True, temperature=0.9, top_p=0.95, repetition_penalty=1.3, seed=5)
    prompts = ["1 2 3", "4 5 6 7", "9 8 7 6 5"]
    together = _run_requests(prompts, **kw)
    for p in prompts:
        alone = _run_requests([p], **kw)
        assert alone[p] == together[p], p


def test_prefill_through_bucket_graphs_gives_the_same_tokens():
    """Packed prompt batches replayed from the graph of their (batch, token) bucket (padding entries take the missing
    rows and tokens, write no K/V and sample into the spare sampler slot) produce the tokens of the eager prefill."""
    kw = dict(max_tokens=12, ignore_eos=True, temperature=0.0)
    os.environ["MSTAR_PREFILL_GRAPHS"] = "0"
    try:
        ref, _ = _tokens(1, True, **kw)
    finally:
        os.environ.pop("MSTAR_PREFILL_GRAPHS", None)
    os.environ["MSTAR_EMULATE_GRAPHS"] = "1"
    os.environ["MSTAR_DECODE_BURST"] = "1"
    try:
        cfg = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 256},
               "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
        s = APIServer(cfg, in_process=True).start(60)
        try:
            rids = [s.submit_request(p, output_modalities=["text"], model_kwargs=dict(kw)) for p in ("1 2 3", "7 8 9 10 11")]
            got = [b"".join(c.data for c in s.collect_results(r, 120)["text"]).decode().split() for r in rids]
            eng = s.deployment.workers[0].engines.engine_for("LLM")
            assert eng.prefill_graph_hits >= 1
            assert any(len(k) == 4 for k in eng._graphs), list(eng._graphs)       # a (node, walk, batch, tokens) bucket
        finally:
            s.shutdown()
    finally:
        os.environ.pop("MSTAR_EMULATE_GRAPHS", None)
        os.environ.pop("MSTAR_DECODE_BURST", None)
    assert got == ref
