"""Piecewise CUDA graphs: a forward is cut into pieces; pieces whose tensor shapes repeat are captured once per
shape signature and replayed, the glue between them (data-dependent indexing, host decisions) stays eager.

``PiecewiseCudaGraphRunner.run(name, fn, *tensors)`` is the whole interface: the first call with a new signature
warms ``fn`` up and captures it over static copies of the inputs; later calls copy the inputs in and replay. On the
CPU, or when capture is switched off, ``fn`` simply runs. Outputs of a replay are views of the graph's static output
buffers: valid until the same piece runs again with the same signature.

Reference counterpart: ``PiecewiseCudaGraphRunner`` (mstar/engine/cuda_graph_runner.py; configured by V-JEPA2
mstar/model/vjepa2/submodules.py:919-953 and Qwen3-TTS mstar/model/qwen3_tts/submodules.py:685-715;
signature test test/modular/test_piecewise_config_signature.py).
"""
from __future__ import annotations

import torch


def signature(name: str, tensors) -> tuple:
    return (name,) + tuple((tuple(t.shape), str(t.dtype), t.device.index) for t in tensors)


class PiecewiseCudaGraphRunner:
    def __init__(self, enabled: bool | None = None, max_graphs: int = 64):
        self.enabled = torch.cuda.is_available() if enabled is None else (enabled and torch.cuda.is_available())
        self.max_graphs = max_graphs
        self._graphs: dict[tuple, tuple] = {}
        self.stats = {"captures": 0, "replays": 0, "eager": 0}

    def run(self, name: str, fn, *tensors: torch.Tensor):
        if not self.enabled or not all(t.is_cuda for t in tensors):
            self.stats["eager"] += 1
            return fn(*tensors)
        sig = signature(name, tensors)
        entry = self._graphs.get(sig)
        if entry is None:
            if len(self._graphs) >= self.max_graphs:
                self.stats["eager"] += 1
                return fn(*tensors)
            static_in = [t.clone() for t in tensors]
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
            self.stats["captures"] += 1
        g, static_in, static_out = entry
        for dst, src in zip(static_in, tensors):
            dst.copy_(src)
        g.replay()
        self.stats["replays"] += 1
        return static_out
