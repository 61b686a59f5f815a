"""Builds the engines of a worker: one KV-cache engine per AR node group, one stateless engine per flavor of
stateless nodes, with the node group's tensor / sequence parallel groups.

Reference counterpart: ``EngineManager.build`` / ``warmup_all`` (mstar/worker/engine_manager.py:68-237).
"""
from __future__ import annotations

import torch

from ..engine.kv_cache_engine import KVCacheEngine
from ..engine.stateless_engine import StatelessEngine, make_audio_codec_config, make_enc_dec_config
from ..models.base import EngineType


# KV engines of this process by (worker id, node): the decode side of a prefill / decode split pulls pages from the
# prefill side's pool through this table when both live in one process
_KV_ENGINES: dict[tuple[str, str], object] = {}


def register_kv_engines(worker_id: str, manager: "EngineManager") -> None:
    for node, eng in manager.node_to_engine.items():
        if isinstance(eng, KVCacheEngine):
            _KV_ENGINES[(worker_id, node)] = eng


def lookup_kv_engine(worker_id: str, node: str):
    return _KV_ENGINES.get((worker_id, node))


class EngineManager:
    def __init__(self, model, device, node_names: list[str], *, tp_group=None, sp_group=None, kv_overrides=None,
                 max_batch: int = 64, use_cuda_graphs: bool | None = None):
        self.model, self.device = model, torch.device(device)
        self.node_to_engine: dict[str, object] = {}
        self.engines: list = []
        types = model.get_node_engine_types()
        kv_cfgs = {tuple(sorted(c.nodes)): c for c in model.get_kv_cache_config()}
        shards = (tp_group.size if tp_group is not None else 1) * (sp_group.size if sp_group is not None else 1)
        kv_nodes = [n for n in node_names if types.get(n) == EngineType.KV_CACHE]
        done: set[str] = set()
        for nodes_key, cfg in kv_cfgs.items():
            mine = [n for n in nodes_key if n in kv_nodes]
            if not mine:
                continue
            cfg = cfg.shard(shards) if shards > 1 else cfg
            for k, v in (kv_overrides or {}).items():
                if hasattr(cfg, k):
                    setattr(cfg, k, v)
            sub_info = model.get_engine_hints(mine[0]) if hasattr(model, "get_engine_hints") else {}
            eng = KVCacheEngine(mine, self.device, cfg, vocab_size=sub_info.get("vocab_size", 32000),
                                max_batch=sub_info.get("max_batch", max_batch),
                                max_tokens=sub_info.get("max_tokens", 16384),
                                n_pos_axes=sub_info.get("n_pos_axes", 1), group=sub_info.get("group", 1),
                                use_cuda_graphs=use_cuda_graphs, tp_group=tp_group,
                                track_seen=sub_info.get("track_seen", True),
                                decode_burst=int(sub_info.get("decode_burst", 1)))
            eng.load_model(model, tp_group=tp_group, sp_group=sp_group)
            self.engines.append(eng)
            for n in mine:
                self.node_to_engine[n] = eng
                done.add(n)
        by_flavor: dict[str, list[str]] = {}
        for n in node_names:
            if n in done:
                continue
            sub = model.get_submodule(n, self.device, tp_group=tp_group, autocast_dtype=model.get_autocast_dtype(),
                                      sp_group=sp_group)
            by_flavor.setdefault(sub.get_stateless_flavor(), []).append((n, sub))
        for flavor, items in by_flavor.items():
            cfg = make_audio_codec_config() if flavor == "audio_codec" else make_enc_dec_config()
            eng = StatelessEngine([n for n, _ in items], self.device, cfg, tp_group=tp_group)
            for n, sub in items:
                eng.submodules[n] = sub
                self.node_to_engine[n] = eng
            self.engines.append(eng)

    def engine_for(self, node: str):
        return self.node_to_engine[node]

    def warmup_all(self) -> None:
        for e in self.engines:
            e.warmup()

    def remove_request(self, request_id: str) -> None:
        for e in self.engines:
            e.remove_request(request_id)
