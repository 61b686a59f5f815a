"""Control-plane messages between the API server, the conductor and the workers. Plain dataclasses (picklable and
msgpack-able through ``asdict``); the transport underneath is the C++ shared-memory mesh or an in-process queue.

Reference counterpart: mstar/utils/ipc_format.py (worker-bound NEW_REQUEST / REMOVE_REQUEST / INPUT_SIGNALS /
TENSOR_RECEIVED / UNPERSIST_TENSORS / STOP_LOOPS / SCHEDULE_TP, conductor-bound NEW_REQUEST / WORKER_GRAPHS_DONE /
SETUP_DONE / ABORT_REQUEST / FAIL_REQUESTS) and mstar/api_server/request_types.py (API-bound results).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, IntEnum

from ..graph.ir import GraphEdge, TensorPointerInfo


class WorkerMessageType(str, Enum):
    NEW_REQUEST = "new_request"
    REMOVE_REQUEST = "remove_request"
    INPUT_SIGNALS = "input_signals"
    UNPERSIST_TENSORS = "unpersist"
    TENSOR_RECEIVED = "tensor_received"
    TENSOR_RECEIVED_BATCH = "tensor_received_batch"
    SCHEDULE_TP = "schedule_tp"
    STOP_LOOPS = "stop_loops"
    SHUTDOWN = "shutdown"
    HEARTBEAT = "heartbeat"
    KV_EXPORT = "kv_export"          # decode-side worker -> prefill-side worker: send me this request's pages
    KV_IMPORT = "kv_import"          # prefill-side worker -> decode-side worker: descriptors of the packed pages


class ConductorMessageType(str, Enum):
    NEW_REQUEST = "new_request"
    WORKER_GRAPHS_DONE = "worker_graphs_done"
    SETUP_DONE = "setup_done"
    ABORT_REQUEST = "abort_request"
    FAIL_REQUESTS = "fail_requests"
    HEARTBEAT = "heartbeat"
    SHUTDOWN = "shutdown"


class ApiMessageType(str, Enum):
    RESULT_TENSORS = "result_tensors"
    RESULT_TENSORS_BATCH = "result_tensors_batch"    # the client-bound outputs of one executed batch, all requests
    REQUEST_COMPLETE = "request_complete"
    REQUEST_FAILED = "request_failed"
    SETUP_DONE = "setup_done"


class MessageSource(IntEnum):
    CONDUCTOR = 0
    TP_RANK_0 = 1
    SELF = 2


@dataclass
class SamplingParams:
    temperature: float = 0.6
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    ignore_eos: bool = False


@dataclass
class CurrentForwardPassInfo:
    """What a worker needs to know about the walk it is asked to run for a request."""
    request_id: str
    graph_walk: str
    requires_cfg: bool = False
    fwd_index: int = 0
    random_seed: int = 0
    max_tokens: int = 2048
    sampling_config: dict = field(default_factory=dict)     # name -> SamplingParams fields ("main", aux names)
    step_metadata: dict = field(default_factory=dict)
    per_label_seq_info: dict = field(default_factory=dict)  # label -> (seq_len, next_position)
    partition_name: str = "default"
    loop_stop_times: dict = field(default_factory=dict)
    dynamic_loop_iter_counts: dict = field(default_factory=dict)   # loop name -> max_iters override


@dataclass
class NewRequest:
    request_id: str
    partition_worker_graph_ids: list[str]
    worker_graph_to_workers: dict[str, list[str]]
    initial_inputs: list[GraphEdge]
    request_info: CurrentForwardPassInfo


@dataclass
class RemoveRequest:
    request_id: str
    source: int = MessageSource.CONDUCTOR


@dataclass
class InputSignals:
    request_id: str
    inputs: list[GraphEdge]
    request_info: CurrentForwardPassInfo | None = None
    partition_name: str = "default"
    producer_done: set = field(default_factory=set)


@dataclass
class TensorReceived:
    request_id: str
    successful_tensors: dict[str, int] = field(default_factory=dict)
    failed_tensor_ids: list[str] = field(default_factory=list)


@dataclass
class KVExport:
    request_id: str
    node_name: str
    reply_to: str


@dataclass
class KVImport:
    request_id: str
    node_name: str
    source_worker: str
    meta: dict = field(default_factory=dict)
    tensor_info: dict = field(default_factory=dict)      # name -> TensorPointerInfo


@dataclass
class UnpersistTensors:
    request_id: str
    uuid_to_ref_count: dict[str, int] = field(default_factory=dict)


@dataclass
class StopLoops:
    request_id: str
    loop_names: set
    partition_name: str = "default"
    loop_stop_times: dict = field(default_factory=dict)


@dataclass
class ScheduleTPNode:
    node_name: str
    graph_walk: str
    request_ids: list[str]


@dataclass
class NewRequestConductor:
    request_id: str
    initial_signals: dict[str, list[TensorPointerInfo]]
    initial_input_modalities: list[str]
    initial_output_modalities: list[str]
    input_metadata: dict = field(default_factory=dict)
    model_kwargs: dict = field(default_factory=dict)


@dataclass
class WorkerGraphsDone:
    request_id: str
    worker_graph_ids: list[str]
    is_first_tp_rank: bool = True
    persist_signals: dict[str, list[TensorPointerInfo]] = field(default_factory=dict)
    new_token_counts: dict[str, int] = field(default_factory=dict)
    per_label_seq_info: dict = field(default_factory=dict)
    partition_name: str = "default"
    partition_done: bool = False
    stream_tokens_consumed: dict[str, int] = field(default_factory=dict)
    output_loop_indices: dict = field(default_factory=dict)
    timings: dict = field(default_factory=dict)
    walk: str = ""


@dataclass
class SetupDone:
    worker_id: str


@dataclass
class AbortRequest:
    request_id: str


@dataclass
class FailRequests:
    """request_id -> error message; one step can fail several requests for different reasons."""
    errors: dict[str, str]
    status: int = 500


@dataclass
class ResultTensors:
    request_id: str
    modality: str
    tensors: list[TensorPointerInfo]
    metadata: dict = field(default_factory=dict)
    source_entity: str = ""


@dataclass
class ResultTensorsBatch:
    items: list[ResultTensors] = field(default_factory=list)


@dataclass
class TensorReceivedBatch:
    items: list = field(default_factory=list)      # TensorReceived records


@dataclass
class RequestComplete:
    request_id: str
    final_outputs: dict = field(default_factory=dict)
    profile: dict = field(default_factory=dict)


@dataclass
class RequestFailed:
    request_id: str
    error_message: str
    status: int = 500


@dataclass
class Message:
    """Envelope: ``type`` is one of the enums above, ``body`` the matching dataclass, ``src`` the sender."""
    type: str
    body: object = None
    src: str = ""
