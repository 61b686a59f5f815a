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


def test_arena_block_larger_than_a_segment_gets_its_own_segment():
    name = _prefix()
    ar = ShmArena(name, segment_bytes=1 << 20, max_segments=3)
    r = ShmArenaReader()
    try:
        big = torch.arange(3 << 18, dtype=torch.float32)          # 3 MB against 1 MB segments
        seg, off = ar.write("big", big)
        assert seg == 1
        v = r.view(name, seg, off, big.numel() * 4, torch.float32, big.shape)
        assert torch.equal(v, big)
        ar.write("small", torch.zeros(1000))                      # regular blocks still go to the regular segments
        assert ar.free("big")
    finally:
        r.close()
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


def test_arena_segments_are_registered_with_cuda_within_the_pin_budget():
    """``cudaHostRegister`` of arena segments, driven against counting stand-ins for the two CUDA runtime calls:
    the first segment is pinned, a segment added by growth is pinned while the budget lasts, later ones stay
    pageable, consumers pin the segments they map, and everything is unregistered on close."""
    import ctypes
    import uuid

    import torch

    from mstar_b200.communication.arena import ShmArena, ShmArenaReader, _bind
    from mstar_b200.ops import _lib
    lib = _bind(_lib.runtime())
    calls = {"reg": [], "unreg": []}
    REG = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint)
    UNREG = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
    reg = REG(lambda p, n, flags: calls["reg"].append((p, n, flags)) or 0)
    unreg = UNREG(lambda p: calls["unreg"].append(p) or 0)
    lib.mstar_arena_set_pin_hooks(ctypes.cast(reg, ctypes.c_void_p), ctypes.cast(unreg, ctypes.c_void_p))
    try:
        seg = 1 << 20
        a = ShmArena("t_pin_" + uuid.uuid4().hex[:8], segment_bytes=seg, max_segments=3)
        assert a.pin(budget_bytes=2 * seg) == 1 and a.pinned_bytes == seg
        assert calls["reg"][0][1] == seg and calls["reg"][0][2] == 1          # whole segment, portable flag
        blob = torch.arange(200_000, dtype=torch.float32)                      # 800 KB: three of them need 3 segments
        locs = [a.write(f"u{i}", blob + i) for i in range(3)]
        assert a.num_segments == 3 and a.pinned_bytes == 2 * seg and len(calls["reg"]) == 2
        r = ShmArenaReader(pin=True)
        v = r.view(a.base_name, locs[2][0], locs[2][1], blob.numel() * 4, torch.float32, blob.shape)
        assert torch.equal(v, blob + 2) and r.pinned_segments == 1 and len(calls["reg"]) == 3
        r.close()
        a.close()
        assert len(calls["unreg"]) == 3
    finally:
        lib.mstar_arena_set_pin_hooks(None, None)
