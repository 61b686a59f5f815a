"""C++ host runtime: shared-memory mesh (mailboxes, wake-ups, cross-process delivery) and the arena allocator
(coalescing, segment growth, canaries, cross-process zero-copy reads)."""
import multiprocessing as mp
import os
import threading
import time
import uuid

import pytest
import torch

from mstar_b200.communication.arena import ShmArena, ShmArenaReader, sweep_orphans
from mstar_b200.communication.communicator import LocalCommunicator, ShmMeshCommunicator
from mstar_b200.utils.ipc_format import AbortRequest, Message


def _prefix():
    return "mstartest_" + uuid.uuid4().hex[:8]


def test_local_communicator_roundtrip():
    hub = LocalCommunicator.new_hub()
    a, b = LocalCommunicator("a", hub), LocalCommunicator("b", hub)
    a.send("b", Message("abort_request", AbortRequest("r1")))
    got = b.recv_or_wake(0.5)
    assert len(got) == 1 and got[0].body.request_id == "r1" and got[0].src == "a"
    assert b.drain() == []
    b.wake()
    assert b.recv_or_wake(0.5) == []


def test_mesh_send_drain_order_and_wrap():
    p = _prefix()
    a, b = ShmMeshCommunicator("a", p, ring_bytes=16384), ShmMeshCommunicator("b", p, ring_bytes=16384)
    try:
        n = 400                      # ~400 * 200 B wraps a 16 KB ring many times
        got = []
        for i in range(n):
            a.send("b", Message("x", {"i": i, "pad": "p" * 100}))
            if i % 7 == 0:
                got += b.drain()
        got += b.drain()
        assert [m.body["i"] for m in got] == list(range(n))
    finally:
        a.close(); b.close()


def test_mesh_recv_blocks_until_message_or_wake():
    p = _prefix()
    a, b = ShmMeshCommunicator("a", p), ShmMeshCommunicator("b", p)
    try:
        t0 = time.time()
        assert b.recv_or_wake(0.15) == [] and time.time() - t0 >= 0.1
        threading.Timer(0.05, lambda: a.send("b", Message("hi", 1))).start()
        t0 = time.time()
        got = b.recv_or_wake(2.0)
        assert len(got) == 1 and time.time() - t0 < 1.0
        threading.Timer(0.05, b.wake).start()
        t0 = time.time()
        assert b.recv_or_wake(2.0) == [] and time.time() - t0 < 1.0
        big = "z" * (3 << 20)       # larger than the default receive buffer
        a.send("b", Message("big", big))
        assert b.recv_or_wake(1.0)[0].body == big
    finally:
        a.close(); b.close()


def _child_sender(prefix, n):
    c = ShmMeshCommunicator("child", prefix)
    for i in range(n):
        c.send("parent", Message("n", i))
    c.close()


def test_mesh_cross_process_many_producers():
    p = _prefix()
    parent = ShmMeshCommunicator("parent", p)
    try:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_child_sender, args=(p, 200)) for _ in range(1)]
        for pr in procs:
            pr.start()
        got = []
        deadline = time.time() + 60
        while len(got) < 200 and time.time() < deadline:
            got += parent.recv_or_wake(0.2)
        for pr in procs:
            pr.join(30)
        assert [m.body for m in got] == list(range(200))
    finally:
        parent.close()


def test_arena_alloc_free_coalesce_and_growth():
    name = _prefix()
    ar = ShmArena(name, segment_bytes=1 << 20, max_segments=3)
    try:
        ts = {f"t{i}": torch.full((40000,), float(i)) for i in range(5)}     # 160 KB each
        for k, t in ts.items():
            ar.write(k, t)
        used = ar.bytes_in_use
        assert used >= 5 * 160000
        ar.free("t1"); ar.free("t2")
        assert ar.largest_free(0) >= 2 * 160000          # neighbours coalesced
        ar.free("t0")
        assert ar.largest_free(0) >= 3 * 160000
        for i in range(10):                               # forces more segments
            ar.write(f"g{i}", torch.zeros(50000))
        assert ar.num_segments >= 2
        with pytest.raises(MemoryError):
            for i in range(100):
                ar.write(f"h{i}", torch.zeros(60000))
    finally:
        ar.close()


def _child_reader(name, seg, off, nbytes, q):
    r = ShmArenaReader()
    v = r.view(name, seg, off, nbytes, torch.float32, (nbytes // 4,))
    q.put(float(v.sum()))
    r.close()


def test_arena_cross_process_zero_copy_and_canary():
    name = _prefix()
    ar = ShmArena(name, segment_bytes=1 << 20)
    try:
        t = torch.arange(1000, dtype=torch.float32)
        seg, off = ar.write("u", t)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        pr = ctx.Process(target=_child_reader, args=(name, seg, off, 4000, q))
        pr.start()
        assert q.get(timeout=60) == float(t.sum())
        pr.join(30)
        # overwrite past the end of the block: the canary check on free must notice
        r = ShmArenaReader()
        v = r.view(name, seg, off, 4096 + 64, torch.uint8, (4096 + 64,))
        v[4096:] = 7
        with pytest.raises(RuntimeError):
            ar.free("u")
        r.close()
    finally:
        ar.close()
    assert sweep_orphans(name) == 0
