"""Per-node executable unit. An engine drives a submodule through
``prepare_inputs -> preprocess -> forward / forward_batched -> postprocess -> check_stop``.

Reference counterparts: ``NodeInputs`` / ``ARNodeInputs`` (mstar/model/submodule_base.py:23-130),
``PerRequestState`` (:133-184), ``ModelInputsFromEngine`` (:187-218), ``NodeSubmodule`` (:221-465),
``ARNodeSubmodule`` (:468-530).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

BATCHED_LOGITS = "__batched_logits__"     # output key: the engine samples from it


@dataclass
class NodeInputs:
    request_id: str
    graph_walk: str
    tensor_inputs: dict[str, list[torch.Tensor]] = field(default_factory=dict)
    kwargs: dict = field(default_factory=dict)


@dataclass
class ARNodeInputs(NodeInputs):
    input_seq_len: int = 0
    input_ids: torch.Tensor | None = None
    input_embeds: torch.Tensor | None = None
    custom_pos_ids: torch.Tensor | None = None


@dataclass
class PerRequestState:
    """Scratch that a submodule keeps for a request across forwards (scheduler state, step counters, ...)."""
    request_id: str
    data: dict = field(default_factory=dict)


@dataclass
class ModelInputsFromEngine:
    request_ids: list[str]
    per_request_info: dict           # request_id -> CurrentForwardPassInfo
    cache_manager: object = None     # BatchedCacheManager for KV engines
    batch_context: object = None     # BatchContext planned by the engine
    preallocated_buffers: dict = field(default_factory=dict)
    sampler: object = None
    per_request_states: dict = field(default_factory=dict)


class NodeSubmodule:
    """Stateless (encoder / decoder / codec / DiT step) node. Override what the node needs."""

    node_name: str = ""

    def __init__(self, device="cpu", dtype=torch.bfloat16):
        self.device, self.dtype = torch.device(device), dtype

    # -- per request --
    def prepare_inputs(self, graph_walk: str, fwd_info, inputs: dict[str, list[torch.Tensor]]) -> NodeInputs:
        return NodeInputs(fwd_info.request_id, graph_walk, inputs, dict(fwd_info.step_metadata or {}))

    def preprocess(self, graph_walk: str, engine_inputs: ModelInputsFromEngine, inputs: list[NodeInputs]) -> dict:
        return {}

    def forward(self, graph_walk: str, engine_inputs: ModelInputsFromEngine, node_inputs: NodeInputs, **kw) -> dict:
        raise NotImplementedError

    def forward_batched(self, graph_walk: str, engine_inputs: ModelInputsFromEngine, inputs: list[NodeInputs],
                        **kw) -> list[dict]:
        return [self.forward(graph_walk, engine_inputs, ni, **kw) for ni in inputs]

    def postprocess(self, request_id: str, request_info, outputs: dict, inputs: NodeInputs) -> dict:
        """Map raw forward outputs to named output tensors (edge name -> tensor)."""
        return outputs

    def check_stop(self, request_id: str, request_info, outputs: dict) -> set[str]:
        """Names of loops that should stop after this iteration."""
        return set()

    # -- batching / graphs --
    def can_batch(self, graph_walk: str) -> bool:
        return True

    def max_batch_size(self, graph_walk: str) -> int:
        return 64

    def get_stateless_flavor(self) -> str:
        return "enc_dec"

    def get_cuda_graph_configs(self) -> list:
        return []

    def can_use_cuda_graphs(self, graph_walk: str) -> bool:
        return False

    def can_graph_prefill(self, graph_walk: str) -> bool:
        """Multi-token (prefill) batches of this walk may be replayed from a captured graph over (batch, token)
        buckets: ``forward_graph`` must then work from the static id buffer alone for any packed batch (no per-request
        tensors, no host-side row surgery)."""
        return False

    def cleanup_request(self, request_id: str) -> None:
        pass

    def load_weights(self, model_dir: str | None) -> None:
        pass


class ARNodeSubmodule(NodeSubmodule):
    """Autoregressive node backed by the paged KV pool."""

    def get_needed_cache_labels(self, graph_walk: str, fwd_info) -> list[str]:
        return ["main"]

    def prepare_inputs(self, graph_walk: str, fwd_info, inputs: dict[str, list[torch.Tensor]]) -> ARNodeInputs:
        ids = None
        for key in ("input_ids", "tok", "new_token"):
            ts = inputs.get(key)
            if ts:
                # one tensor (every decode step): no concatenation kernel, no copy
                ids = ts[0].reshape(-1) if len(ts) == 1 else torch.cat([t.reshape(-1) for t in ts])
                if ids.dtype != torch.int64:
                    ids = ids.to(torch.int64)
                break
        return ARNodeInputs(fwd_info.request_id, graph_walk, inputs, dict(fwd_info.step_metadata or {}),
                            input_seq_len=0 if ids is None else int(ids.numel()), input_ids=ids)

    def first_stop_index(self, request_id: str, request_info, tokens: list[int]) -> int | None:
        """Index of the first token of a decode burst at which ``check_stop`` asks for a stop, or None. Nodes with a
        plain stop-token rule override this with something cheaper than one ``check_stop`` call per token."""
        for j, t in enumerate(tokens):
            if self.check_stop(request_id, request_info, {"new_token_host": t}):
                return j
        return None

    def filter_batched_output(self, outputs: dict, row: int) -> dict:
        return {k: (v[row] if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in outputs.items()}

    def unpack_packed_outputs(self, outputs: dict, q_lens: list[int]) -> list[dict]:
        return [self.filter_batched_output(outputs, i) for i in range(len(q_lens))]
