"""Engine for nodes without a KV cache: encoders, VAE / codec decoders, DiT steps, combine nodes. Batches the
ready requests through ``forward_batched`` and can replay captured CUDA graphs for fixed shapes.

Reference counterparts: ``StatelessEngineConfig`` / ``make_enc_dec_config`` / ``make_audio_codec_config`` and
``StatelessEngine`` (mstar/engine/stateless_engine.py:42-650), ``StatelessCudaGraphRunner``
(mstar/engine/cuda_graph_runner.py:2025-2348).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models.submodule_base import ModelInputsFromEngine
from .base import BaseEngine, NodeOutput, PreparedBatch


@dataclass
class StatelessEngineConfig:
    flavor: str = "enc_dec"                         # enc_dec | audio_codec
    max_batch_size: int = 16
    capture_batch_sizes: list[int] = field(default_factory=lambda: [1, 2, 4, 8, 16])
    use_cuda_graphs: bool = False
    dtype: torch.dtype = torch.bfloat16


def make_enc_dec_config(**kw) -> StatelessEngineConfig:
    return StatelessEngineConfig(flavor="enc_dec", **kw)


def make_audio_codec_config(**kw) -> StatelessEngineConfig:
    kw.setdefault("dtype", torch.float32)
    return StatelessEngineConfig(flavor="audio_codec", **kw)


class StatelessCudaGraphRunner:
    """Captures ``fn(*static_inputs)`` once per shape signature and replays it with inputs copied into the static
    buffers. Outputs are views of static buffers: callers clone what they keep."""

    def __init__(self):
        self._graphs: dict = {}

    def run(self, key, fn, inputs: list[torch.Tensor]):
        sig = (key, tuple((tuple(t.shape), t.dtype) for t in inputs))
        entry = self._graphs.get(sig)
        if entry is None:
            static_in = [t.clone() for t in inputs]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    fn(*static_in)
                s.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                    static_out = fn(*static_in)
            torch.cuda.current_stream().wait_stream(s)
            entry = (g, static_in, static_out)
            self._graphs[sig] = entry
        g, static_in, static_out = entry
        for dst, src in zip(static_in, inputs):
            dst.copy_(src)
        g.replay()
        return static_out


class StatelessEngine(BaseEngine):
    def __init__(self, node_names, device, config: StatelessEngineConfig | None = None, tp_group=None):
        super().__init__(node_names, device)
        self.config = config or StatelessEngineConfig()
        self.tp_group = tp_group
        self.graph_runner = StatelessCudaGraphRunner() if self.device.type == "cuda" else None
        self.states: dict[str, dict] = {}

    def execute_forward(self, planned: PreparedBatch):
        b = planned.batch
        sub = self.submodules[b.node_name]
        if self.tp_group is not None and getattr(self.tp_group, "symm", None) is not None:
            self.tp_group.symm.barrier()       # device-side arrival flags instead of a host barrier per forward
        ei = ModelInputsFromEngine(planned.request_ids, b.fwd_infos,
                                   per_request_states={r: self.states.setdefault(r, {}) for r in planned.request_ids},
                                   preallocated_buffers={"graph_runner": self.graph_runner})
        with torch.no_grad():
            sub.preprocess(b.graph_walk, ei, planned.node_inputs)
            if sub.can_batch(b.graph_walk) and len(planned.node_inputs) > 1:
                return sub.forward_batched(b.graph_walk, ei, planned.node_inputs)
            return [sub.forward(b.graph_walk, ei, ni) for ni in planned.node_inputs]

    def postprocess(self, planned: PreparedBatch, raw, out: NodeOutput) -> None:
        b = planned.batch
        sub = self.submodules[b.node_name]
        for rid, ni, r in zip(planned.request_ids, planned.node_inputs, raw):
            try:
                out.outputs[rid] = sub.postprocess(rid, b.fwd_infos[rid], r, ni)
                stops = sub.check_stop(rid, b.fwd_infos[rid], out.outputs[rid])
                if stops:
                    out.stop_loops[rid] = set(stops)
            except Exception as e:  # noqa: BLE001
                out.failed_requests[rid] = f"postprocess failed: {e!r}"

    def remove_request(self, request_id: str) -> None:
        self.states.pop(request_id, None)
        super().remove_request(request_id)
