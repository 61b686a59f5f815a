from .chunk_policy import ChunkPolicy, FixedChunkPolicy, LeftContextChunkPolicy, SlidingWindowChunkPolicy
from .stream_buffer import StreamBuffer, StreamChunk
from .topology import Connection, PartitionDefinition, PartitionTopology, StreamingGraphEdge

__all__ = ["ChunkPolicy", "FixedChunkPolicy", "LeftContextChunkPolicy", "SlidingWindowChunkPolicy", "StreamBuffer",
           "StreamChunk", "Connection", "PartitionDefinition", "PartitionTopology", "StreamingGraphEdge"]
