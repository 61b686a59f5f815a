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

    def can_graph_prefill(self, graph_walk):
        return type(self).forward_batched is DecoderSubmodule.forward_batched      # plain token prompts only

    def postprocess(self, request_id, request_info, outputs, inputs):
        tok = outputs["new_token"].to(torch.int64)          # device view: feeds the next step
        host = outputs.get("new_token_host")
        # what leaves the node (client, stream buffers of other partitions) is a host tensor: the value was read back
        # with the batch anyway, and consumers then never issue per-token device ops
        if outputs.get("burst_host_tensor") is not None:    # a decode burst: all of its tokens leave together
            out_tok = outputs["burst_host_tensor"]          # int64 host view of the batch's read-back, no copy
        elif outputs.get("burst_host") is not None:
            out_tok = torch.tensor([int(t) for t in outputs["burst_host"]], dtype=torch.int64)
        else:
            out_tok = torch.tensor([int(host)], dtype=torch.int64) if host is not None else tok
        return {self.token_edge: out_tok, "tok": tok, "last_token": tok}

    def check_stop(self, request_id, request_info, outputs):
        sc = (request_info.sampling_config or {}).get("main", {})
        if not sc.get("ignore_eos", False) and outputs.get("new_token_host") in self.eos_ids:
            return {self.loop_name}
        return set()

    def first_stop_index(self, request_id, request_info, tokens):
        sc = (request_info.sampling_config or {}).get("main", {})
        if sc.get("ignore_eos", False) or not self.eos_ids:
            return None
        eos = self.eos_ids
        return next((j for j, t in enumerate(tokens) if t in eos), None)


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


class MultimodalDecoderSubmodule(DecoderSubmodule):
    """Decoder LM whose prompt carries placeholder token ids that are replaced, row by row and in order, by
    encoder features (audio frames, image patches) before the prefill forward. ``placeholders`` maps an input
    edge name to the token id that marks its rows. Optional ``position_fn(ids, inputs, kwargs) -> int32 [3, T]``
    supplies multi-axis rotary positions (and the position the decode continues from via ``pos_delta``).

    Reference counterparts: the per-modality prefill walks of Qwen3-Omni (mstar/model/qwen3_omni/submodules.py,
    prefill_text / prefill_audio / prefill_vision), Higgs-Audio (mstar/model/higgs_audio/submodules.py) and
    BAGEL's ViT prefill (mstar/model/bagel/submodules.py); merged here into one packed prefill forward.
    """

    def __init__(self, lm, device, placeholders: dict[str, int], eos_ids=(), loop_name="decode_loop",
                 token_edge="new_token", position_fn=None, emit_hidden: str | None = None,
                 deepstack: dict[str, int] | None = None):
        """``deepstack``: edge name -> number of tapped encoder layers whose features ride in the same rows, after
        the main features (row width (1 + taps) x hidden); they are added to the first decoder layers' outputs."""
        super().__init__(lm, device, eos_ids=eos_ids, loop_name=loop_name, token_edge=token_edge)
        self.placeholders, self.position_fn, self.emit_hidden = dict(placeholders), position_fn, emit_hidden
        self.deepstack = dict(deepstack or {})

    def prepare_inputs(self, graph_walk, fwd_info, inputs):
        ni = super().prepare_inputs(graph_walk, fwd_info, inputs)
        if self.position_fn is not None and ni.input_ids is not None and ni.input_ids.numel() > 1:
            pos, delta = self.position_fn(ni.input_ids, inputs, ni.kwargs)
            ni.custom_pos_ids = pos
            ni.kwargs["_pos_delta"] = int(delta)
        return ni

    def preprocess(self, graph_walk, engine_inputs, inputs):
        cm = engine_inputs.cache_manager
        for ni in inputs:       # decode continues from the largest multimodal position, not from the token count
            d = ni.kwargs.pop("_pos_delta", None)
            if d is not None and cm is not None:
                cm.set_custom_pos_advance(ni.request_id, "main", d)
        return {}

    def forward_batched(self, graph_walk, engine_inputs, inputs, **kw):
        ids = torch.cat([ni.input_ids.reshape(-1) for ni in inputs]).to(self.device)
        x = self.lm.embed(ids)
        H, off = x.shape[-1], 0
        deep_rows, deep_feats = [], []
        for ni in inputs:
            n = ni.input_ids.numel()
            for edge, pid in self.placeholders.items():
                feats = ni.tensor_inputs.get(edge)
                if not feats:
                    continue
                taps = self.deepstack.get(edge, 0)
                f = torch.cat([t.reshape(-1, H * (1 + taps)) for t in feats]).to(self.device, x.dtype)
                rows = (ids[off:off + n] == pid).nonzero().reshape(-1) + off
                if rows.numel() != f.shape[0]:
                    raise ValueError(f"{edge}: {f.shape[0]} feature rows for {rows.numel()} placeholder tokens")
                x[rows] = f[:, :H]
                if taps:
                    deep_rows.append(rows)
                    deep_feats.append(f[:, H:].reshape(-1, taps, H))
            off += n
        deep = None
        if deep_rows:
            d = torch.cat(deep_feats)
            deep = (torch.cat(deep_rows), [d[:, k].contiguous() for k in range(d.shape[1])])
        out = self.lm(engine_inputs.batch_context, inputs_embeds=x, return_hidden=self.emit_hidden is not None,
                      deepstack=deep)
        if self.emit_hidden is None:
            return {BATCHED_LOGITS: out}
        logits, hidden = out
        return {BATCHED_LOGITS: logits, self.emit_hidden: hidden.index_select(0, engine_inputs.batch_context.logit_rows)}

    def forward_graph(self, graph_walk, engine_inputs, static_ids, ctx):
        if self.emit_hidden is None:
            return {BATCHED_LOGITS: self.lm(ctx, input_ids=static_ids)}
        logits, hidden = self.lm(ctx, input_ids=static_ids, return_hidden=True)
        return {BATCHED_LOGITS: logits, self.emit_hidden: hidden.index_select(0, ctx.logit_rows)}

    def postprocess(self, request_id, request_info, outputs, inputs):
        out = super().postprocess(request_id, request_info, outputs, inputs)
        if self.emit_hidden is not None and self.emit_hidden in outputs:
            out[self.emit_hidden] = outputs[self.emit_hidden].reshape(1, -1)
        return out


def expand_placeholders(ids: list[int], placeholder: int, counts: list[int]) -> list[int]:
    """Replace the i-th occurrence of ``placeholder`` by ``counts[i]`` copies of it."""
    out, i = [], 0
    for t in ids:
        if t == placeholder and i < len(counts):
            out.extend([placeholder] * counts[i])
            i += 1
        else:
            out.append(t)
    return out
