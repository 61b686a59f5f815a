"""When does a stream buffer hold enough items for its consumer, and how far does a pop advance?

Reference counterparts: ``ChunkPolicy``, ``SlidingWindowChunkPolicy``, ``LeftContextChunkPolicy``,
``FixedChunkPolicy`` (mstar/streaming/chunk_policy.py:4-152).
"""
from __future__ import annotations


class ChunkPolicy:
    """Contract: ``is_ready(n)`` — n buffered items suffice; ``window_size()`` — items handed to the consumer;
    ``next_chunk_size(n)`` — items the read position advances by (smaller than the window for overlapping
    policies)."""

    def __init__(self):
        self.first_chunk_read = False
        self.items_consumed = 0

    def register_chunk(self, advanced_by: int) -> None:
        self.first_chunk_read = True
        self.items_consumed += advanced_by

    def is_ready(self, buffer_len: int) -> bool:
        raise NotImplementedError

    def next_chunk_size(self, buffer_len: int) -> int:
        raise NotImplementedError

    def window_size(self) -> int:
        raise NotImplementedError

    def continue_after_producer_done(self) -> bool:
        """True: after the producer has finished and the buffer is drained, keep handing out empty chunks; the
        consumer decides by itself when it is done (a talker that keeps speaking after the thinker's EOS)."""
        return False


class SlidingWindowChunkPolicy(ChunkPolicy):
    """``window`` items per chunk, advancing by ``stride`` (Orpheus -> SNAC: window 28 tokens, stride 7)."""

    def __init__(self, window: int, stride: int):
        super().__init__()
        if stride <= 0 or window < stride:
            raise ValueError("need 0 < stride <= window")
        self.window, self.stride = window, stride

    def is_ready(self, buffer_len):
        return buffer_len >= self.window

    def next_chunk_size(self, buffer_len):
        return self.stride

    def window_size(self):
        return self.window


class LeftContextChunkPolicy(ChunkPolicy):
    """Chunks of ``chunk`` new items preceded by ``left_context`` already-seen items (streaming vocoders that warm
    up on overlap). The first chunk has no context; to leave its tail in the buffer as the second chunk's
    context, the first pop advances by ``chunk - left_context`` only."""

    def __init__(self, chunk: int, left_context: int):
        super().__init__()
        if left_context >= chunk:
            raise ValueError("left_context must be smaller than chunk")
        self.chunk, self.left_context = chunk, left_context

    def is_ready(self, buffer_len):
        return buffer_len >= (self.chunk + self.left_context if self.first_chunk_read else self.chunk)

    def next_chunk_size(self, buffer_len):
        return self.chunk if self.first_chunk_read else self.chunk - self.left_context

    def window_size(self):
        return self.chunk + self.left_context if self.first_chunk_read else self.chunk


class FixedChunkPolicy(ChunkPolicy):
    """Non-overlapping chunks of ``chunk_size`` items."""

    def __init__(self, chunk_size: int, continue_after_done: bool = False):
        super().__init__()
        self.chunk_size, self._continue = chunk_size, continue_after_done

    def is_ready(self, buffer_len):
        return buffer_len >= self.chunk_size

    def next_chunk_size(self, buffer_len):
        return self.chunk_size

    def window_size(self):
        return self.chunk_size

    def continue_after_producer_done(self):
        return self._continue
