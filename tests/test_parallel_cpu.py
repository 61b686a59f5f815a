"""Host-side parallel logic on CPU: mesh rank math, sharded-edge fan-out / fan-in, sequence splits, and gloo
ranks running the collective wrappers and Ulysses exchange."""
import os
import subprocess
import sys

import torch

from mstar_b200.graph.ir import GraphEdge, TensorPointerInfo
from mstar_b200.models.base import WorkerGraph, divide_into_worker_graphs
from mstar_b200.parallel.comm import GlobalParallelConfig
from mstar_b200.parallel.sequence_parallel import sp_seq_split
from mstar_b200.parallel.sharding import ShardingConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mesh_rank_math():
    wg = WorkerGraph("g", ["dit"], [4, 5, 6, 7], tp_size=2, sp_size=2)
    assert wg.tp_ranks(4) == [4, 5] and wg.tp_ranks(7) == [6, 7]
    assert wg.sp_ranks(4) == [4, 6] and wg.sp_ranks(5) == [5, 7]
    cfg = GlobalParallelConfig([0, 1, 2, 3, 4, 5, 6, 7], tp_size=2, sp_size=2)
    assert cfg.instances() == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert cfg.tp_groups() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert cfg.sp_groups() == [[0, 2], [1, 3], [4, 6], [5, 7]]
    wgs = divide_into_worker_graphs([{"node_names": ["LLM"], "ranks": [0, 1, 2, 3], "tp_size": 2}])
    assert [w.ranks for w in wgs] == [[0, 1], [2, 3]] and wgs[0].group_id == wgs[1].group_id


def test_sharding_fanout_matched_and_mismatched():
    sc = ShardingConfig({"hidden": 0})
    assert sc.compute_fanout("tok", 2, 4) == [[(0, 0.0, 1.0)], [(1, 0.0, 1.0)], [(0, 0.0, 1.0)], [(1, 0.0, 1.0)]]
    assert sc.compute_fanout("hidden", 2, 2) == [[(0, 0.0, 1.0)], [(1, 0.0, 1.0)]]
    up = sc.compute_fanout("hidden", 2, 4)       # each source shard is cut in two
    assert up[0] == [(0, 0.0, 0.5)] and up[1] == [(0, 0.5, 1.0)] and up[3] == [(1, 0.5, 1.0)]
    down = sc.compute_fanout("hidden", 4, 2)     # each destination reads two whole source shards
    assert down[0] == [(0, 0.0, 1.0), (1, 0.0, 1.0)] and sc.compute_fanin("hidden", 4, 2) == 2
    shards = [[TensorPointerInfo([8, 16], "bfloat16", 256, uuid=f"s{r}")] for r in range(2)]
    edges = sc.fanout_graph_edges(GraphEdge("dit", "hidden"), shards, 4)
    assert [e.tensor_info[0].offset for e in edges] == [0, 128, 0, 128]
    assert [e.tensor_info[0].dims for e in edges] == [[4, 16]] * 4


def test_sequence_split_is_balanced():
    assert sp_seq_split(10, 4) == [0, 3, 6, 8, 10]
    assert sp_seq_split(8, 2) == [0, 4, 8]


def test_gloo_ranks_collectives_and_ulysses():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", "2", os.path.join(ROOT, "tests", "mp_cpu_worker.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
