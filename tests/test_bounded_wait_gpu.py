"""A device-side wait that nobody answers gives up after its limit, reports where through the status word, and leaves
the kernel through its normal exit: the context stays usable and the next kernel computes correctly.

The missing peer is made on the host: a two-rank peer table whose second "rank" is plain local memory that nothing
ever signals. No fault, trap or endless loop is involved: the wait limit is set to one millisecond for the call and
restored afterwards."""
import ctypes

import pytest
import torch

from mstar_b200.ops import _lib, gemm

pytestmark = pytest.mark.gpu

KID_COMM, PHASE_BARRIER = 5, 4
MAX_RANKS = 8


@pytest.mark.expects_status
def test_unanswered_peer_barrier_times_out_reports_and_the_next_gemm_is_correct():
    lib = _lib.kernels()
    dev = torch.device("cuda")
    assert _lib.read_status(clear=True)[0] == 0
    data = [torch.zeros(256, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(16 * MAX_RANKS, dtype=torch.int32, device=dev) for _ in range(2)]     # [channel][rank] words
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    Ptrs = ctypes.c_void_p * MAX_RANKS
    bufs = Ptrs(*([d.data_ptr() for d in data] + [None] * (MAX_RANKS - 2)))
    flgs = Ptrs(*([f.data_ptr() for f in flags] + [None] * (MAX_RANKS - 2)))
    channel = 3
    old = lib.mstar_get_wait_limit_ns()
    _lib.set_wait_limit_ns(1_000_000)                      # 1 ms
    try:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        rc = lib.mstar_peer_barrier(bufs, flgs, 2, 0, ctypes.c_void_p(state.data_ptr()), channel,
                                    ctypes.c_void_p(_lib.stream_ptr()))
        end.record()
        assert rc == 0, lib.mstar_last_error()
        torch.cuda.synchronize()                           # returns: the kernel left by itself
        assert start.elapsed_time(end) < 500.0             # about the limit, nowhere near the 2 s default
    finally:
        _lib.set_wait_limit_ns(old)
    code, block, aux0, aux1 = _lib.read_status(clear=True)
    assert code == (KID_COMM << 16 | PHASE_BARRIER), hex(code)
    assert (block, aux0, aux1) == (0, 1, channel)          # gave up waiting for rank 1 on that channel
    assert int(flags[1][channel * MAX_RANKS + 0]) == 1     # its own signal went out before it waited
    assert _lib.read_status(clear=True)[0] == 0            # cleared by the read above
    # the context is intact: a tensor-core GEMM right after the timeout matches its fp32 oracle
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 1024, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(512, 1024, generator=g) * 0.05).to(torch.bfloat16).cuda()
    got, ref = gemm.linear(x, w), gemm.linear_ref(x, w)
    torch.cuda.synchronize()
    assert (got.float() - ref.float()).abs().max().item() <= 2e-2 * max(1.0, ref.float().abs().max().item())
    assert _lib.read_status(clear=True)[0] == 0


@pytest.mark.expects_status
def test_status_travels_with_a_serving_batch():
    """The asynchronous copy used by the engines sees the same word as the synchronous read."""
    lib = _lib.kernels()
    dev = torch.device("cuda")
    _lib.read_status(clear=True)
    pinned = torch.zeros(4, dtype=torch.int32).pin_memory()
    _lib.status_copy_async(pinned)
    torch.cuda.synchronize()
    assert pinned.tolist() == [0, 0, 0, 0]
    data = [torch.zeros(256, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(16 * MAX_RANKS, dtype=torch.int32, device=dev) for _ in range(2)]
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    Ptrs = ctypes.c_void_p * MAX_RANKS
    bufs = Ptrs(*([d.data_ptr() for d in data] + [None] * (MAX_RANKS - 2)))
    flgs = Ptrs(*([f.data_ptr() for f in flags] + [None] * (MAX_RANKS - 2)))
    old = lib.mstar_get_wait_limit_ns()
    _lib.set_wait_limit_ns(1_000_000)
    try:
        assert lib.mstar_peer_barrier(bufs, flgs, 2, 0, ctypes.c_void_p(state.data_ptr()), 0,
                                      ctypes.c_void_p(_lib.stream_ptr())) == 0
        _lib.status_copy_async(pinned)
        torch.cuda.synchronize()
    finally:
        _lib.set_wait_limit_ns(old)
    assert int(pinned[0]) == (KID_COMM << 16 | PHASE_BARRIER) and int(pinned[2]) == 1
    assert "collective wait ran out in phase 4" in _lib.decode_status(int(pinned[0]))
    assert _lib.read_status(clear=True)[0] == int(pinned[0])
