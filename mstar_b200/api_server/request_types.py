"""API-side request records. Reference counterpart: mstar/api_server/request_types.py."""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field


@dataclass
class ResultChunk:
    modality: str                 # text | audio | image | video | error
    data: bytes = b""
    metadata: dict = field(default_factory=dict)
    final: bool = False
    error_status: int | None = None


@dataclass
class PendingRequest:
    request_id: str
    output_modalities: list[str]
    model_kwargs: dict
    chunks: "queue.Queue[ResultChunk]" = field(default_factory=queue.Queue)
    done: bool = False
    wake: object = None                 # callable set by an event-loop consumer parked on an empty queue
    sink: object = None                 # callable(ResultChunk): chunks bypass the queue and go straight to the transport
    lock: threading.Lock = field(default_factory=threading.Lock, repr=False)
    t_submit: float = field(default_factory=time.time)
    t_first_chunk: float | None = None
    t_last_chunk: float | None = None
    t_preprocessed: float | None = None
    inputs: dict = field(default_factory=dict)        # modality -> [count, bytes]
    outputs: dict = field(default_factory=dict)       # modality -> [count, bytes]
    profile: dict = field(default_factory=dict)
