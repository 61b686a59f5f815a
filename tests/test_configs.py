"""Every deployment file under ``configs/``: parses, names a registered model, places every node that its walks
need, forms whole tensor- / sequence-parallel instances, and gives the conductor a worker graph for every walk."""
import glob
import os

import pytest
import yaml

from mstar_b200.communication.communicator import LocalCommunicator
from mstar_b200.conductor.conductor import Conductor
from mstar_b200.conductor.deployment import load_config
from mstar_b200.models.registry import get_model_class

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
FILES = sorted(glob.glob(os.path.join(ROOT, "*.yaml")))


def test_the_reference_deployments_all_have_a_counterpart():
    names = {os.path.basename(f) for f in FILES}
    for want in ("bagel.yaml", "bagel_cfg_parallel.yaml", "bagel_img_disaggregated.yaml", "bagel_pd_disaggregated.yaml",
                 "bagel_single_gpu.yaml", "cosmos3_droid.yaml", "cosmos3_nano.yaml", "cosmos3_nano_sp2.yaml",
                 "cosmos3_nano_sp4.yaml", "cosmos3_nano_tp2.yaml", "cosmos3_nano_tp2_sp2.yaml", "cosmos3_nano_tp4.yaml",
                 "cosmos3_super_tp2.yaml", "cosmos3_super_tp2_sp2.yaml", "cosmos3_super_tp4.yaml", "higgs_audio.yaml",
                 "orpheus.yaml", "orpheus_colocated.yaml", "orpheus_pd_disaggregated.yaml", "orpheus_tp2.yaml",
                 "pi05.yaml", "pi05_droid.yaml", "qwen3_omni.yaml", "qwen3_omni_2gpu.yaml", "qwen3_omni_colocated.yaml",
                 "qwen3_omni_full_tp2.yaml", "qwen3_omni_pd_disaggregated.yaml", "qwen3_omni_thinker_tp2.yaml",
                 "qwen3_tts.yaml", "vjepa2.yaml", "vjepa2_ac.yaml", "wan22.yaml", "whisper_large.yaml"):
        assert want in names, want


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f) for f in FILES])
def test_config_places_every_walk(path):
    with open(path) as f:
        raw = yaml.safe_load(f)
    cfg = load_config(path)
    assert cfg["model"] == raw["model"] and cfg["node_groups"]
    kw = dict(cfg.get("model_kwargs") or {})
    kw.update(small=True) if cfg["model"] != "tiny" else None
    model = get_model_class(cfg["model"])(model_dir=None, skip_weight_loading=True, **kw)
    wgs = model.get_worker_graphs(cfg["node_groups"])
    placed = {n for wg in wgs for n in wg.node_names}
    optional = set(model.get_optional_nodes()) if hasattr(model, "get_optional_nodes") else set()
    walks = model.get_graph_walk_graphs()
    known = set()
    for w in walks.values():
        known |= set(_nodes(w))
    assert placed <= known, f"nodes that no walk uses: {sorted(placed - known)}"
    assert known - placed <= optional, f"unplaced nodes: {sorted(known - placed - optional)}"
    for wg in wgs:
        assert len(wg.ranks) == wg.tp_size * wg.sp_size
        for w in wg.graph_walks or []:
            assert w in walks, f"{w!r} is not a walk of {cfg['model']}"
    cond = Conductor(cfg, model, LocalCommunicator("conductor", LocalCommunicator.new_hub()))
    for name, w in walks.items():
        needed = set(_nodes(w))
        if needed - placed:              # a walk of optional nodes that this deployment leaves out
            assert needed - placed <= optional
            continue
        serving = [wg for wg in wgs if wg.serves(name) and set(wg.node_names) & needed]
        assert serving, f"no group serves walk {name!r}"
        for n in needed:                 # every node of the walk has a group that serves the walk
            assert any(n in wg.node_names for wg in serving), (name, n)
    assert cond.worker_graphs


def _nodes(section):
    from mstar_b200.graph.ir import GraphNode
    if isinstance(section, GraphNode):
        return [section.name]
    out = []
    for attr in ("sections", "body", "section"):
        v = getattr(section, attr, None)
        if v is None:
            continue
        for s in (v if isinstance(v, (list, tuple)) else [v]):
            out += _nodes(s)
    return out


def test_qwen3_omni_placements_give_the_same_answer():
    """One GPU, two GPUs, colocated groups and prompt / decode disaggregation of the thinker: the same text and the
    same amount of speech for a request with audio and image input (test-sized weights, in-process ranks)."""
    import torch
    from mstar_b200.api_server.server import APIServer

    def run(name):
        cfg = load_config(os.path.join(ROOT, name))
        cfg.update(model_kwargs=dict(cfg.get("model_kwargs") or {}, small=True), use_cuda_graphs=False)
        torch.manual_seed(0)
        s = APIServer(cfg, in_process=True).start(120)
        try:
            kw = dict(max_tokens=6, ignore_eos=True, temperature=0.0, max_audio_tokens=12)
            tens = {"audio": [torch.randn(8000, generator=torch.Generator().manual_seed(1)) * 0.1],
                    "image": [torch.rand(3, 16, 16, generator=torch.Generator().manual_seed(2))]}
            r = s.collect_results(s.submit_request("describe", output_modalities=["text", "audio"], model_kwargs=kw,
                                                   tensors=tens), 120)
            assert "error" not in r, r
            return b"".join(c.data for c in r["text"]), sum(len(c.data) for c in r["audio"])
        finally:
            s.shutdown()
    want = run("qwen3_omni.yaml")
    assert len(want[0].split()) == 6 and want[1] > 0
    for name in ("qwen3_omni_colocated.yaml", "qwen3_omni_2gpu.yaml", "qwen3_omni_pd_disaggregated.yaml"):
        assert run(name) == want, name
