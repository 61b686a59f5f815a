"""Multi-process deployment on CPU: conductor and worker as OS processes over the C++ shared-memory mesh and
arena; worker-death detection through heartbeats (the failure is made on the host: the worker process is
terminated between requests)."""
import time

import pytest

from mstar_b200.api_server.server import APIServer
from mstar_b200.models import tiny

CFG = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128}, "use_cuda_graphs": False,
       "node_groups": [{"node_names": ["LLM"], "ranks": [0]}]}


def _tokens(res):
    return [int(t) for t in b"".join(c.data for c in res["text"]).decode().split()]


def test_processes_over_shm_mesh_and_worker_death(monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    s = APIServer(CFG, in_process=False, heartbeat_s=0.2, heartbeat_timeout_s=1.5).start(180)
    try:
        model = tiny.build_tiny()
        prompts = tiny.synthetic_prompts(n=2, lo=8, hi=12, seed=21)
        ref = tiny.oracle_generate(model, prompts, 5)
        rids = [s.submit_request(" ".join(map(str, p)), model_kwargs=dict(max_tokens=5, temperature=0.0)) for p in prompts]
        outs = [_tokens(s.collect_results(r, 120)) for r in rids]
        assert outs == ref
        # host-made failure: the worker process goes away while idle
        worker_proc = s.deployment.procs[1]
        worker_proc.terminate()
        worker_proc.join(10)
        rid = s.submit_request("1 2 3", model_kwargs=dict(max_tokens=50, temperature=0.0))
        res = s.collect_results(rid, 30)
        assert "error" in res and res["error"][0].error_status == 503
        assert b"stopped responding" in res["error"][0].data
    finally:
        s.shutdown()


def test_prefill_decode_split_across_processes_moves_the_kv_pages(monkeypatch):
    """Prefill worker and decode worker as separate OS processes with separate page pools: the decode side asks the
    prefill side for the request's pages (packed into one tensor per label, carried by the shared-memory arena
    between CPU processes; a CUDA IPC handle between GPU processes) and produces the colocated run's tokens."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    base = {"model": "tiny", "model_kwargs": {"dtype": "float32", "max_num_pages": 128}, "use_cuda_graphs": False}
    pd = dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0], "graph_walks": ["prefill"]},
                                 {"node_names": ["LLM"], "ranks": [1], "graph_walks": ["decode"]}])
    co = dict(base, node_groups=[{"node_names": ["LLM"], "ranks": [0]}])
    outs = []
    for cfg in (co, pd):
        s = APIServer(cfg, in_process=False, heartbeat_s=0.5, heartbeat_timeout_s=20).start(180)
        try:
            rids = [s.submit_request(f"{i} 2 3 4 5 6 7 8 9", model_kwargs=dict(max_tokens=10, temperature=0.7, top_p=0.9,
                                                                              repetition_penalty=1.2, seed=5 + i))
                    for i in range(3)]
            res = [s.collect_results(r, 120) for r in rids]
            assert all("error" not in r for r in res), res
            outs.append([_tokens(r) for r in res])
        finally:
            s.shutdown()
    assert all(len(t) == 10 for t in outs[0]) and outs[0] == outs[1]
