"""The per-request profile: workers report node timings (launch / in flight / post) and tensor transfers with every
finished walk, the API server merges them with its own timestamps and byte counts and renders the tree."""
from mstar_b200.api_server.server import APIServer
from mstar_b200.profile.display import format_profile, render
from mstar_b200.profile.records import RequestProfile, WorkerProfile


def test_worker_profile_accumulates_and_merges():
    wp = WorkerProfile("worker_0")
    wp.record_batch("LLM", "decode", ["a", "b"], launch_s=0.002, flight_s=0.030, post_s=0.004, iterations={"a": 7, "b": 7},
                    speculative=True)
    wp.record_batch("LLM", "decode", ["a"], launch_s=0.001, flight_s=0.020, post_s=0.002, iterations={"a": 3})
    wp.record_transfer("a", "tx", "audio", "worker_0", "api", 4096, 0.0001)
    d = wp.pop("a")
    assert wp.pop("a") == {"nodes": [], "transfers": []}
    rp = RequestProfile("a", checkpoints={"received": 0.0, "first_chunk": 0.1, "finished": 0.5})
    rp.merge_worker(d)
    rp.merge_worker(d)              # a second walk's report of the same node adds up
    nt = rp.nodes[0]
    assert (nt.executions, nt.iterations, nt.speculative, nt.batch_rows) == (4, 20, 2, 6)
    assert abs(nt.post_s - 2 * (0.002 + 0.002)) < 1e-9
    assert rp.transfers[0].count == 2 and rp.transfers[0].nbytes == 8192
    text = render(RequestProfile.from_dict(rp.to_dict()))
    assert "LLM @ worker_0" in text and "2 speculative" in text and "worker_0 -> api" in text and "timeline" in text


def test_server_builds_the_profile_of_a_served_request(tmp_path):
    out = tmp_path / "stats.txt"
    cfg = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 64},
           "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}
    s = APIServer(cfg, in_process=True, log_stats_file=str(out)).start(60)
    try:
        rid = s.submit_request("1 2 3", model_kwargs=dict(max_tokens=6, temperature=0.0))
        res = s.collect_results(rid, 60)
        assert "error" not in res
        rp = s.request_profile(s.pending[rid])
    finally:
        s.shutdown()
    walks = {(n.node, n.walk) for n in rp.nodes}
    assert ("LLM", "prefill") in walks and ("LLM", "decode") in walks
    dec = next(n for n in rp.nodes if n.walk == "decode")
    assert dec.iterations == 5 and dec.flight_s > 0 and dec.launch_s > 0
    assert rp.outputs["text"][0] == 6 and rp.inputs["text"][0] == 1
    assert rp.checkpoints["first_chunk"] <= rp.checkpoints["last_chunk"] <= rp.checkpoints["finished"]
    text = out.read_text()
    assert f"request {rid}" in text and "nodes:" in text
    # the bare conductor summary still renders (no worker profiles attached)
    assert "timeline" in format_profile("x", {"queue_s": 0.001, "total_s": 0.2, "tokens_out": 3, "walks": []})
