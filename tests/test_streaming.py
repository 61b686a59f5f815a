"""Chunk policies and the stream buffer: windows, strides, left context, out-of-order arrival, final flush."""
import torch

from mstar_b200.streaming import (FixedChunkPolicy, LeftContextChunkPolicy, SlidingWindowChunkPolicy, StreamBuffer)


def _buf(policy):
    return StreamBuffer("r", "codes", "llm", policy)


def test_sliding_window_28_7():
    b = _buf(SlidingWindowChunkPolicy(28, 7))
    for i in range(27):
        b.put(f"t{i}", torch.tensor(i))
    assert not b.has_chunk_ready()
    b.put("t27", torch.tensor(27))
    assert b.has_chunk_ready()
    c = b.pop_chunk()
    assert c.data["data"].tolist() == list(range(28)) and c.start_offset == 0 and not c.is_final
    assert not b.has_chunk_ready()
    for i in range(28, 35):
        b.put(f"t{i}", torch.tensor(i))
    c = b.pop_chunk()
    assert c.data["data"].tolist() == list(range(7, 35)) and c.start_offset == 7 and c.chunk_index == 1


def test_out_of_order_payloads_wait_for_their_turn():
    b = _buf(FixedChunkPolicy(2))
    b.pre_read_register("a")
    b.pre_read_register("b")
    b.put("b", torch.tensor(2))
    assert not b.has_chunk_ready()
    b.put("a", torch.tensor(1))
    assert b.has_chunk_ready() and b.pop_chunk().data["data"].tolist() == [1, 2]


def test_final_flush_partial_and_empty():
    b = _buf(FixedChunkPolicy(4))
    for i in range(6):
        b.put(f"t{i}", torch.tensor(i))
    assert b.pop_chunk().data["data"].tolist() == [0, 1, 2, 3]
    assert not b.has_chunk_ready()
    b.signal_done()
    assert b.has_chunk_ready()
    c = b.pop_chunk()
    assert c.data["data"].tolist() == [4, 5] and c.is_final
    assert not b.has_chunk_ready()
    # producer finishes exactly on a chunk boundary: one empty final chunk closes the stream, once
    b2 = _buf(FixedChunkPolicy(2))
    b2.put("x", torch.tensor(1)); b2.put("y", torch.tensor(2))
    assert not b2.pop_chunk().is_final
    b2.signal_done()
    assert b2.has_chunk_ready()
    c = b2.pop_chunk()
    assert c.data["data"] is None and c.is_final
    assert not b2.has_chunk_ready()


def test_left_context_policy():
    b = _buf(LeftContextChunkPolicy(chunk=4, left_context=2))
    for i in range(10):
        b.put(f"t{i}", torch.tensor(i))
    c0 = b.pop_chunk()
    assert c0.data["data"].tolist() == [0, 1, 2, 3] and c0.start_offset == 0
    c1 = b.pop_chunk()
    assert c1.data["data"].tolist() == [2, 3, 4, 5, 6, 7] and c1.start_offset == 2
    assert not b.has_chunk_ready()


def test_continue_after_producer_done_never_final():
    b = _buf(FixedChunkPolicy(2, continue_after_done=True))
    b.put("x", torch.tensor(1))
    b.signal_done()
    c = b.pop_chunk()
    assert c.data["data"].tolist() == 1 or c.data["data"].tolist() == [1]
    assert not c.is_final and b.has_chunk_ready()
    assert b.pop_chunk().data["data"] is None
