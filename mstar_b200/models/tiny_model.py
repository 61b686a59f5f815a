"""``tiny``: the 2-layer Qwen-style decoder as a served model (standing fixture of the framework tests and the
CPU smoke configuration). Token ids in, token ids out: prompts are space-separated ids or raw bytes."""
from __future__ import annotations

import torch

from ..engine.kv_store import KVCacheConfig
from .base import EngineType, Model
from .llm_common import DecoderSubmodule, LMStateMachine, lm_walks
from .tiny import build_tiny, tiny_config


class TinyLM(Model):
    name = "tiny"

    def __init__(self, model_dir=None, skip_weight_loading=False, dtype: str | None = None, page_size: int = 16,
                 max_num_pages: int = 256, **kw):
        super().__init__(model_dir, skip_weight_loading, **kw)
        self.dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, None: None}[dtype]
        self.page_size, self.max_num_pages = page_size, max_num_pages
        self.cfg = tiny_config()
        self.sm = LMStateMachine()

    def get_graph_walk_graphs(self):
        return lm_walks()

    def get_node_engine_types(self):
        return {"LLM": EngineType.KV_CACHE}

    def get_kv_cache_config(self):
        c = self.cfg
        return [KVCacheConfig(c.num_layers, c.num_kv_heads, c.head_dim, max_seq_len=4096,
                              max_num_pages=self.max_num_pages, page_size=self.page_size, num_qo_heads=c.num_heads,
                              nodes=["LLM"], dtype=self._dtype_for(None))]

    def _dtype_for(self, device):
        if self.dtype is not None:
            return self.dtype
        return torch.bfloat16 if torch.cuda.is_available() else torch.float32

    def get_default_sharding_config(self):
        return {"LLM": {"tp": True, "sp": False}}

    def get_engine_hints(self, node):
        c = self.cfg
        return dict(vocab_size=c.vocab_size, group=c.num_heads // c.num_kv_heads, max_tokens=4096)

    def get_autocast_dtype(self):
        return self._dtype_for(None)

    def get_submodule(self, node_name, device, tp_group=None, autocast_dtype=None, sp_group=None):
        lm = build_tiny(device=device, dtype=self._dtype_for(device), tp=tp_group).fold_norms()
        return DecoderSubmodule(lm, device, eos_ids=self.model_kwargs.get("eos_ids", ()))

    def process_prompt(self, prompt, input_modalities, output_modalities, tensors, **kw):
        parts = (prompt or "").split()
        if parts and all(p.isdigit() for p in parts):
            ids = [int(p) % self.cfg.vocab_size for p in parts]
        else:
            ids = list((prompt or " ").encode("utf-8"))
        return {"input_ids": [torch.tensor(ids, dtype=torch.int64)]}

    def get_initial_forward_pass_args(self, partition_name, input_modalities, output_modalities, input_signals,
                                      model_kwargs):
        return self.sm.initial(input_signals, self.get_max_output_tokens(model_kwargs))

    def get_partition_forward_pass_args(self, partition_name, partition_metadata, persist_signals,
                                        incoming_connections=None):
        return self.sm.next(partition_metadata, persist_signals)

    def postprocess(self, output, modality, request_kwargs):
        ids = output.reshape(-1).tolist() if isinstance(output, torch.Tensor) else list(output)
        return (" ".join(str(int(i)) for i in ids) + " ").encode()
