"""Shared pieces of the decoder-LM backed models: the AR submodule that runs a ``DecoderLM`` under the KV-cache
engine, the two-walk (prefill, decode loop) graph, and the conductor-side state machine that chains them.

Reference counterparts: Orpheus walks and state machine (mstar/model/orpheus/orpheus_model.py:111-281) and its LLM
submodule with in-graph sampling (mstar/model/orpheus/submodules.py).
"""
from __future__ import annotations

import torch

from ..graph.ir import EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, Loop
from .base import ForwardPassArgs
from .submodule_base import ARNodeSubmodule, BATCHED_LOGITS


class DecoderSubmodule(ARNodeSubmodule):
    def __init__(self, lm, device, eos_ids=(), loop_name="decode_loop", token_edge="new_token"):
        super().__init__(device, lm.cfg.dtype)
        self.lm, self.eos_ids, self.loop_name, self.token_edge = lm, set(eos_ids), loop_name, token_edge

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ids = torch.cat([ni.input_ids.reshape(-1) for ni in inputs]).to(self.device)
        return {BATCHED_LOGITS: self.lm(engine_inputs.batch_context, input_ids=ids)}

    def forward_graph(self, graph_walk, engine_inputs, static_ids, ctx):
        """Capturable decode step: ids come from the engine's static buffer, the plan from the device plan slot."""
        return {BATCHED_LOGITS: self.lm(ctx, input_ids=static_ids)}

    def can_use_cuda_graphs(self, graph_walk):
        return True

    def postprocess(self, request_id, request_info, outputs, inputs):
        tok = outputs["new_token"].to(torch.int64)
        return {self.token_edge: tok, "tok": tok, "last_token": tok}

    def check_stop(self, request_id, request_info, outputs):
        sc = (request_info.sampling_config or {}).get("main", {})
        if not sc.get("ignore_eos", False) and outputs.get("new_token_host") in self.eos_ids:
            return {self.loop_name}
        return set()


def lm_walks(node: str = "LLM", loop_name: str = "decode_loop", max_iters: int = 2048, modality: str = "text",
             stream_edge: GraphEdge | None = None, prefill_inputs: set[str] | None = None,
             pre_nodes: list | None = None) -> dict:
    """prefill: one forward over the prompt; decode: a loop that feeds each sampled token back into the node.
    ``pre_nodes`` (encoders whose outputs feed the prefill node as ``prefill_inputs``) run before the prefill."""
    def outs(extra):
        o = [GraphEdge(EMIT_TO_CLIENT, "new_token", output_modality=modality, conductor_new_token=True)] if modality else []
        if stream_edge is not None:
            o.append(stream_edge.clone())
        return o + extra
    prefill = GraphNode(node, {"input_ids"} | set(prefill_inputs or ()),
                        outs([GraphEdge(EMPTY_DESTINATION, "last_token", persist=True)]))
    if pre_nodes:
        from ..graph.ir import Parallel, Sequential
        prefill = Sequential([pre_nodes[0] if len(pre_nodes) == 1 else Parallel(list(pre_nodes)), prefill])
    step = GraphNode(node, {"tok"}, outs([GraphEdge(node, "tok")]))
    return {"prefill": prefill, "decode": Loop(step, max_iters=max_iters, name=loop_name)}


class LMStateMachine:
    """prefill -> decode -> done, shared by the LLM-only models."""

    def __init__(self, node: str = "LLM", loop_name: str = "decode_loop"):
        self.node, self.loop_name = node, loop_name

    def initial(self, input_signals: dict, max_tokens: int, extra_edges: list | None = None) -> ForwardPassArgs:
        return ForwardPassArgs({"graph_walk": "prefill", "max_tokens": max_tokens},
                               [GraphEdge(self.node, "input_ids", list(input_signals.get("input_ids", [])))]
                               + list(extra_edges or []))

    def next(self, metadata: dict, persist: dict) -> ForwardPassArgs:
        budget = metadata["max_tokens"] - metadata["tokens_out"]
        if metadata["finished_walk"] == "prefill" and budget > 0 and persist.get("last_token"):
            last = persist.pop("last_token")
            return ForwardPassArgs({"graph_walk": "decode", "max_tokens": budget,
                                    "dynamic_loop_iter_counts": {self.loop_name: budget}},
                                   [GraphEdge(self.node, "tok", last[-1:])],
                                   unpersist_tensors=[t.uuid for t in last])
        return ForwardPassArgs(request_done=True)
