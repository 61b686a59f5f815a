"""End to end in one process on the CPU: API server core -> conductor -> worker -> KV engine -> tiny decoder,
checked against the cache-free oracle; plus abort, failure propagation and admission."""
import time

import pytest
import torch

from mstar_b200.api_server.server import APIServer
from mstar_b200.models import tiny

CFG = {"model": "tiny", "max_concurrent_requests": 8,
       "model_kwargs": {"dtype": "float32", "page_size": 16, "max_num_pages": 128},
       "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}


@pytest.fixture(scope="module")
def server():
    s = APIServer(CFG, in_process=True).start(60)
    yield s
    s.shutdown()


def _gen(server, prompt_ids, n, **kw):
    rid = server.submit_request(" ".join(map(str, prompt_ids)), model_kwargs=dict(max_tokens=n, temperature=0.0, **kw))
    res = server.collect_results(rid, 120)
    assert "error" not in res, res.get("error")
    text = b"".join(c.data for c in res["text"]).decode()
    return [int(t) for t in text.split()]


def test_generate_matches_oracle(server):
    model = tiny.build_tiny()
    prompts = tiny.synthetic_prompts(n=3, lo=8, hi=24, seed=9)
    ref = tiny.oracle_generate(model, prompts, 8)
    for p, r in zip(prompts, ref):
        assert _gen(server, p, 8) == r


def test_concurrent_requests_batch_together(server):
    model = tiny.build_tiny()
    prompts = tiny.synthetic_prompts(n=6, lo=8, hi=16, seed=11)
    ref = tiny.oracle_generate(model, prompts, 6)
    rids = [server.submit_request(" ".join(map(str, p)), model_kwargs=dict(max_tokens=6, temperature=0.0)) for p in prompts]
    outs = []
    for rid in rids:
        res = server.collect_results(rid, 120)
        outs.append([int(t) for t in b"".join(c.data for c in res["text"]).decode().split()])
    assert outs == ref
    assert server.deployment.conductor.stats["completed"] >= 6


def test_streaming_chunks_arrive_one_token_at_a_time(server):
    rid = server.submit_request("1 2 3 4 5", model_kwargs=dict(max_tokens=5, temperature=0.0))
    chunks = list(server.iter_result_chunks(rid, 60))
    assert len(chunks) == 5 and all(c.modality == "text" for c in chunks)


def test_abort_releases_the_request(server):
    rid = server.submit_request("1 2 3", model_kwargs=dict(max_tokens=2000, temperature=0.0))
    time.sleep(0.3)
    server.abort_request(rid)
    res = server.collect_results(rid, 30)
    assert res["error"][0].error_status == 499
    deadline = time.time() + 10
    w = server.deployment.workers[0]
    while time.time() < deadline and any(k[0] == rid for k in w.requests):
        time.sleep(0.05)
    assert not any(k[0] == rid for k in w.requests)
    assert _gen(server, [5, 6, 7], 3)          # the server still serves


def test_bad_prompt_fails_only_that_request(server):
    rid = server.submit_request(None, files=[("x.unknownext", b"123")], model_kwargs={})
    res = server.collect_results(rid, 30)
    assert res["error"][0].error_status == 400
    assert _gen(server, [9, 9, 9], 2)


def test_kernel_timeout_status_fails_the_batch_and_the_server_goes_on(server):
    """A kernel whose bounded wait ran out reports through the device status word that travels with every batch.
    Made on the host here: the engine's status check answers once as if the word had been set. The requests of that
    batch must fail (no partial tokens delivered as a success) and later requests must be served."""
    eng = server.deployment.workers[0].engines.engine_for("LLM")
    real = eng.check_batch_status
    fired = []

    def once(out):
        if not fired and out.graph_walk == "decode":
            fired.append(1)
            return "device status 0x50001: collective wait ran out in phase 1 (block 0, aux 1, 0)"
        return real(out)
    eng.check_batch_status = once
    try:
        rid = server.submit_request("1 2 3 4", model_kwargs=dict(max_tokens=50, temperature=0.0))
        res = server.collect_results(rid, 60)
        assert "error" in res and "wait ran out" in res["error"][0].data.decode(errors="replace"), res
    finally:
        eng.check_batch_status = real
    assert fired
    assert _gen(server, [4, 4, 4], 3)
