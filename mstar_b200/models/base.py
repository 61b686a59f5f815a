"""Model contract. A model declares its components (graph nodes), the walks through them, which engine runs each
node, KV-cache needs, default sharding, prompt processing, the conductor-side state machine that decides which
walk follows which, and post-processing of outputs into bytes for the client.

Reference counterparts: ``WorkerGraph`` and mesh rank computation (mstar/model/base.py:39-93),
``_divide_into_worker_graphs`` (:111-225), ``ForwardPassArgs`` (:228-243), ``Model`` (:246-604), engine types,
``MAX_OUTPUT_TOKENS``.
"""
from __future__ import annotations

import io
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from enum import Enum

import torch

from ..engine.kv_store import KVCacheConfig
from ..graph.ir import GraphEdge, GraphSection, TensorPointerInfo
from ..ops.sampling import MultiSamplingConfig, SamplingConfig
from ..streaming.topology import PartitionDefinition, PartitionTopology

MAX_OUTPUT_TOKENS = 2048
NameToTensorList = dict[str, list[torch.Tensor]]


def small_scale() -> int:
    """Width multiplier of the test-sized model variants: on a GPU they are widened so that every layer has a shape
    the tensor-core kernels accept (64-wide heads, 16-byte aligned rows); on the CPU they stay minimal."""
    return 4 if torch.cuda.is_available() else 1


def seeded_init(build, seed: int = 0):
    """``build()`` under its own generator state: modules that take torch's default random initialisation (codecs,
    autoencoders before a checkpoint is loaded) then get the same weights in every process and replica."""
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        return build()


class EngineType(str, Enum):
    KV_CACHE = "kv_cache"
    STATELESS = "stateless"


@dataclass
class ForwardPassArgs:
    """What the conductor sends out to start (or continue) a request: the walk, its input edges, tensors that
    may now be released, and whether the request is finished."""
    full_metadata: dict = field(default_factory=dict)       # graph_walk, requires_cfg, max_tokens, ...
    inputs: list[GraphEdge] = field(default_factory=list)
    unpersist_tensors: list[str] = field(default_factory=list)
    request_done: bool = False
    step_metadata: dict = field(default_factory=dict)

    @property
    def graph_walk(self) -> str:
        return self.full_metadata.get("graph_walk", "")


@dataclass
class WorkerGraph:
    """The nodes of one node group as placed on one model instance: a [sp][tp] mesh of ranks."""
    graph_id: str
    node_names: list[str]
    ranks: list[int]
    tp_size: int = 1
    sp_size: int = 1
    graph_walks: list[str] | None = None      # None = every walk
    group_id: str = ""                        # replicas of the same node set share a group id

    def tp_ranks(self, rank: int) -> list[int]:
        i = self.ranks.index(rank)
        s = i // self.tp_size
        return self.ranks[s * self.tp_size:(s + 1) * self.tp_size]

    def sp_ranks(self, rank: int) -> list[int]:
        i = self.ranks.index(rank)
        t = i % self.tp_size
        return [self.ranks[s * self.tp_size + t] for s in range(self.sp_size)]

    @property
    def leader(self) -> int:
        return self.ranks[0]

    def serves(self, walk: str) -> bool:
        return self.graph_walks is None or walk in self.graph_walks


def divide_into_worker_graphs(node_groups: list[dict]) -> list[WorkerGraph]:
    """YAML ``node_groups`` -> worker graphs. A group whose rank count is a multiple of tp*sp yields several
    instances (replicas); groups listing the same node names are replicas of each other too."""
    out: list[WorkerGraph] = []
    for gi, g in enumerate(node_groups):
        tp, sp = int(g.get("tp_size", 1)), int(g.get("sp_size", 1))
        ranks = list(g.get("ranks", [0]))
        inst = tp * sp
        if len(ranks) % inst:
            raise ValueError(f"node group {g.get('node_names')}: {len(ranks)} ranks do not form tp {tp} x sp {sp} instances")
        names = list(g["node_names"])
        gid = "+".join(sorted(names))
        for k in range(len(ranks) // inst):
            out.append(WorkerGraph(graph_id=f"g{gi}i{k}", node_names=names, ranks=ranks[k * inst:(k + 1) * inst],
                                   tp_size=tp, sp_size=sp, graph_walks=g.get("graph_walks"), group_id=gid))
    return out


class Model(ABC):
    """Base class of every served model."""

    name: str = "model"

    def __init__(self, model_dir: str | None = None, skip_weight_loading: bool = False, **model_kwargs):
        self.model_dir = model_dir
        self.skip_weight_loading = skip_weight_loading or model_dir is None
        self.model_kwargs = model_kwargs

    # ---- structure ----
    @abstractmethod
    def get_graph_walk_graphs(self) -> dict[str, GraphSection]:
        ...

    @abstractmethod
    def get_node_engine_types(self) -> dict[str, EngineType]:
        ...

    def get_kv_cache_config(self) -> list[KVCacheConfig]:
        return []

    def get_default_sharding_config(self) -> dict:
        return {}

    def get_worker_graphs(self, node_groups: list[dict]) -> list[WorkerGraph]:
        nodes = set()
        for sec in self.get_graph_walk_graphs().values():
            nodes |= set(sec.nodes())
        wgs = divide_into_worker_graphs(node_groups)
        for wg in wgs:
            unknown = set(wg.node_names) - nodes
            if unknown:
                raise ValueError(f"config places unknown nodes {sorted(unknown)}; model has {sorted(nodes)}")
        placed = {n for wg in wgs for n in wg.node_names}
        if nodes - placed - set(self.get_optional_nodes()):
            raise ValueError(f"nodes without placement: {sorted(nodes - placed - set(self.get_optional_nodes()))}")
        return wgs

    def get_optional_nodes(self) -> set[str]:
        """Nodes that only some walks use and a deployment may leave out (a request whose walk needs one is then
        refused with an error that names it)."""
        return set()

    def validate_sharding(self, wg: WorkerGraph) -> None:
        if wg.tp_size * wg.sp_size > 1:
            allowed = self.get_default_sharding_config()
            for n in wg.node_names:
                cap = allowed.get(n, {})
                if wg.tp_size > 1 and not cap.get("tp", False):
                    raise ValueError(f"node {n} of {self.name} does not support tensor parallelism")
                if wg.sp_size > 1 and not cap.get("sp", False):
                    raise ValueError(f"node {n} of {self.name} does not support sequence parallelism")

    # ---- partitions (asynchronously running groups of walks joined by streams) ----
    def get_partition_topology(self) -> PartitionTopology | None:
        return None

    def get_partitions(self) -> list[PartitionDefinition]:
        return [PartitionDefinition("default", list(self.get_graph_walk_graphs()), "", [])]

    # ---- request life cycle (conductor side) ----
    @abstractmethod
    def process_prompt(self, prompt: str | None, input_modalities: list[str], output_modalities: list[str],
                       tensors: NameToTensorList, **kwargs) -> NameToTensorList:
        """Tokenise / preprocess on the API server: named tensors that become the request's initial signals."""

    @abstractmethod
    def get_initial_forward_pass_args(self, partition_name: str, input_modalities: list[str],
                                      output_modalities: list[str], input_signals: dict[str, list[TensorPointerInfo]],
                                      model_kwargs: dict) -> ForwardPassArgs:
        ...

    @abstractmethod
    def get_partition_forward_pass_args(self, partition_name: str, partition_metadata: dict,
                                        persist_signals: dict[str, list[TensorPointerInfo]],
                                        incoming_connections: dict | None = None) -> ForwardPassArgs:
        """Called when a walk of the partition has finished: next walk, or request_done."""

    @abstractmethod
    def postprocess(self, output: torch.Tensor | list, modality: str, request_kwargs: dict) -> bytes:
        ...

    # ---- execution (worker side) ----
    @abstractmethod
    def get_submodule(self, node_name: str, device, tp_group=None, autocast_dtype=None, sp_group=None):
        ...

    # ---- knobs ----
    def get_sampling_config(self, model_kwargs: dict) -> SamplingConfig:
        return SamplingConfig(temperature=float(model_kwargs.get("temperature", 0.6)),
                              top_k=int(model_kwargs.get("top_k", 0)), top_p=float(model_kwargs.get("top_p", 1.0)),
                              repetition_penalty=float(model_kwargs.get("repetition_penalty", 1.0)),
                              ignore_eos=bool(model_kwargs.get("ignore_eos", False)),
                              _seed=model_kwargs.get("seed"))

    def get_aux_sampling_configs(self, model_kwargs: dict) -> dict[str, SamplingConfig]:
        return {}

    def resolve_sampling_configs(self, model_kwargs: dict) -> MultiSamplingConfig:
        return MultiSamplingConfig(self.get_sampling_config(model_kwargs), self.get_aux_sampling_configs(model_kwargs))

    def get_max_output_tokens(self, model_kwargs: dict | None = None) -> int:
        return int((model_kwargs or {}).get("max_tokens", MAX_OUTPUT_TOKENS))

    def get_autocast_dtype(self) -> torch.dtype:
        return torch.bfloat16

    def get_output_sample_rate(self) -> int:
        return 24000

    def get_output_audio_channels(self) -> int:
        return 1

    # ---- text (API server) ----
    TOKENIZER_SUBDIRS = ("", "tokenizer", "text_tokenizer")

    def tokenizer(self):
        """The checkpoint's own tokenizer when ``model_dir`` holds one (Hugging Face tokenizer files in the directory
        or in a ``tokenizer/`` sub-directory), else None: the models then fall back to byte-level ids, which is what
        the random-init deployments of tests and benchmarks use."""
        if not hasattr(self, "_hf_tokenizer"):
            self._hf_tokenizer = None
            if self.model_dir:
                import os
                for sub in self.TOKENIZER_SUBDIRS:
                    d = os.path.join(self.model_dir, sub) if sub else self.model_dir
                    if any(os.path.exists(os.path.join(d, f)) for f in ("tokenizer.json", "tokenizer_config.json",
                                                                        "tokenizer.model", "vocab.json")):
                        try:
                            from transformers import AutoTokenizer
                            self._hf_tokenizer = AutoTokenizer.from_pretrained(d)
                            break
                        except Exception as e:  # noqa: BLE001
                            import logging
                            logging.getLogger("mstar.model").warning("tokenizer under %s not loaded: %s", d, e)
        return self._hf_tokenizer

    def encode_text(self, text: str | None, vocab_size: int, byte_modulus: int | None = None,
                    default: str = "") -> list[int]:
        """Token ids of ``text``: the checkpoint's tokenizer (no special tokens added: the models place their own),
        or UTF-8 bytes folded into ``byte_modulus`` (default: the vocabulary) without one."""
        text = text or default
        tok = self.tokenizer()
        if tok is not None:
            return [int(i) for i in tok(text, add_special_tokens=False)["input_ids"]]
        m = byte_modulus or vocab_size
        return [b % m for b in text.encode("utf-8")]

    def chat_text(self, prompt: str | None, system: str | None = None) -> str:
        """The prompt wrapped in the checkpoint's chat template (user turn + generation prompt) when the tokenizer
        has one; the plain prompt otherwise."""
        tok = self.tokenizer()
        if tok is None or not getattr(tok, "chat_template", None):
            return prompt or ""
        msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt or ""}]
        return tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)

    def decode_text(self, ids) -> bytes:
        """Client-bound form of generated text tokens. With a byte-level BPE tokenizer (GPT-2 / Qwen / Llama-3 /
        Whisper vocabularies) the tokens' own bytes: streamed one token at a time, a multi-byte character split across
        tokens then reaches the client intact instead of as replacement characters. Other tokenizers: decoded text.
        Without a tokenizer: the ids in decimal. Reference: mstar/model/utils.py:331-366."""
        ids = [int(i) for i in ids]
        tok = self.tokenizer()
        if tok is None:
            return (" ".join(str(i) for i in ids) + " ").encode()
        table = self._byte_table(tok)
        if table is not None:
            special = self._special_ids
            raw = bytearray()
            for t in tok.convert_ids_to_tokens([i for i in ids if i not in special]):
                try:
                    raw.extend(table[c] for c in (t or ""))
                except KeyError:                     # an added token written in plain text
                    raw.extend(t.encode("utf-8"))
            return bytes(raw)
        return tok.decode(ids, skip_special_tokens=True).encode("utf-8")

    def _byte_table(self, tok):
        """Character -> byte map of a byte-level BPE vocabulary, or None when the tokenizer is of another kind (probed
        once: such a vocabulary writes a leading space as U+0120)."""
        if not hasattr(self, "_byte_table_cache"):
            self._byte_table_cache, self._special_ids = None, set(getattr(tok, "all_special_ids", []) or [])
            try:
                probe = tok.convert_ids_to_tokens(tok.encode(" a", add_special_tokens=False))
                if probe and probe[0].startswith("\u0120"):
                    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
                    chars, n = keep[:], 0
                    for b in range(256):
                        if b not in keep:
                            keep.append(b)
                            chars.append(256 + n)
                            n += 1
                    self._byte_table_cache = {chr(c): b for b, c in zip(keep, chars)}
            except Exception:  # noqa: BLE001
                self._byte_table_cache = None
        return self._byte_table_cache

    # ---- media loading (API server) ----
    def load_image(self, path_or_bytes) -> torch.Tensor:
        from PIL import Image
        import numpy as np
        img = Image.open(io.BytesIO(path_or_bytes) if isinstance(path_or_bytes, (bytes, bytearray)) else path_or_bytes)
        return torch.from_numpy(np.asarray(img.convert("RGB")).copy()).permute(2, 0, 1).contiguous()

    def load_audio(self, path_or_bytes) -> torch.Tensor:
        from ..api_server.media_io import read_wav
        pcm, _sr = read_wav(path_or_bytes)
        return pcm

    def load_video(self, path_or_bytes) -> torch.Tensor:
        raise NotImplementedError("video decoding needs an ffmpeg-backed loader")
