"""Reference arm of bench.py: the unmodified reference package (installed under ``baseline/_ref``) serving its own
stock single-GPU Orpheus placement through its own launcher and HTTP API, with synthetic weights.

What this harness adds is data only, because the machine has no network: a Hugging Face cache directory that
holds random-init checkpoints in the layouts the reference downloads (Llama-3.2-3B names in safetensors, the SNAC
decoder's ``config.json`` + ``pytorch_model.bin`` created from the reference's own SNAC class, and a byte-level
tokenizer). The server is started with ``python -m mstar.api_server.entrypoint`` and the reference's
``configs/orpheus_colocated.yaml`` (one GPU), or the same file with every rank of the box listed in both node groups
(N GPUs: ranks of a node group without ``tp_size`` are data-parallel replicas in the reference,
mstar/conductor/conductor.py:475-506); 64 concurrent requests per GPU stream audio over ``POST /generate``. The load
generator is the one the other arm uses (``mstar_b200/bench/tts_client.py``: a plain HTTP client, no part of either
server), with the same warm-up: one request, then a short round at full concurrency.

Metric: decode tokens/s of the box = audio tokens produced by all requests inside the measurement window divided
by the window's wall-clock length at the client (the server is a black box; 7 tokens per 2048 samples of 16-bit
audio). The window opens when every request has delivered its first audio chunk (all 64 are decoding) and closes
when the first request finishes. TTFT is the time from submission to the first audio chunk.
"""
from __future__ import annotations

import json
import os
import shutil
import socket
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
METRIC = "decode_tokens_per_s_per_box"
LLM_REPO = "canopylabs/orpheus-3b-0.1-ft"
TOK_REPO = "canopylabs/orpheus-3b-0.1-pretrained"
SNAC_REPO = "hubertsiuzdak/snac_24khz"
STOCK_COLOCATED_YAML = """model: "orpheus"
max_seq_len: 131072
node_groups:
  - node_names: [LLM]
    ranks: [0]
    graph_walks: [prefill, decode]
  - node_names: [snac_decoder]
    ranks: [0]
    graph_walks: [snac_chunk]
"""


def stock_yaml(n_gpus: int) -> str:
    """The reference's colocated Orpheus placement, with every rank listed when the box has more than one GPU."""
    if n_gpus <= 1:
        return STOCK_COLOCATED_YAML
    ranks = ", ".join(str(r) for r in range(n_gpus))
    return STOCK_COLOCATED_YAML.replace("ranks: [0]", f"ranks: [{ranks}]")


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def _snapshot_dir(cache: str, repo: str) -> str:
    d = os.path.join(cache, "models--" + repo.replace("/", "--"))
    os.makedirs(os.path.join(d, "refs"), exist_ok=True)
    with open(os.path.join(d, "refs", "main"), "w") as f:
        f.write("0" * 40)
    snap = os.path.join(d, "snapshots", "0" * 40)
    os.makedirs(snap, exist_ok=True)
    return snap


def build_synthetic_cache(cache: str, device: str = "cuda") -> None:
    """Random-init checkpoints in the layouts the reference's loaders read."""
    import torch
    from safetensors.torch import save_file
    # tokenizer: 256 byte tokens, no merges, plus the special ids the reference's prompt format uses
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    byte_alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(byte_alphabet))}
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    snap = _snapshot_dir(cache, TOK_REPO)
    tok.save(os.path.join(snap, "tokenizer.json"))
    with open(os.path.join(snap, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "model_max_length": 131072}, f)
    # language model: HF Llama names, N(0, 0.02) bf16
    H, L, Hq, Hkv, D, F, V = 3072, 28, 24, 8, 128, 8192, 156940
    g = torch.Generator(device=device).manual_seed(0)

    def rnd(*shape):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()
    snap = _snapshot_dir(cache, LLM_REPO)
    index = {"metadata": {}, "weight_map": {}}
    shard, n = {"model.embed_tokens.weight": rnd(V, H), "lm_head.weight": rnd(V, H),
                "model.norm.weight": torch.ones(H, dtype=torch.bfloat16)}, 0

    def flush():
        nonlocal shard, n
        name = f"model-{n:05d}.safetensors"
        save_file(shard, os.path.join(snap, name))
        for k in shard:
            index["weight_map"][k] = name
        shard, n = {}, n + 1
    flush()
    for i in range(L):
        p = f"model.layers.{i}."
        shard.update({p + "self_attn.q_proj.weight": rnd(Hq * D, H), p + "self_attn.k_proj.weight": rnd(Hkv * D, H),
                      p + "self_attn.v_proj.weight": rnd(Hkv * D, H), p + "self_attn.o_proj.weight": rnd(H, Hq * D),
                      p + "mlp.gate_proj.weight": rnd(F, H), p + "mlp.up_proj.weight": rnd(F, H),
                      p + "mlp.down_proj.weight": rnd(H, F),
                      p + "input_layernorm.weight": torch.ones(H, dtype=torch.bfloat16),
                      p + "post_attention_layernorm.weight": torch.ones(H, dtype=torch.bfloat16)})
        if i % 7 == 6 or i == L - 1:
            flush()
    with open(os.path.join(snap, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    with open(os.path.join(snap, "config.json"), "w") as f:
        json.dump({"architectures": ["LlamaForCausalLM"], "hidden_size": H, "num_hidden_layers": L,
                   "num_attention_heads": Hq, "num_key_value_heads": Hkv, "intermediate_size": F, "vocab_size": V,
                   "head_dim": D, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False,
                   "torch_dtype": "bfloat16", "model_type": "llama"}, f)
    # codec: the reference's own class with its published 24 kHz configuration, random weights
    sys.path.insert(0, REF)
    try:
        from mstar.model.orpheus.components.snac import SNAC
        cfg = {"sampling_rate": 24000, "encoder_dim": 48, "encoder_rates": [2, 4, 8, 8], "decoder_dim": 1024,
               "decoder_rates": [8, 8, 4, 2], "attn_window_size": None, "codebook_size": 4096, "codebook_dim": 8,
               "vq_strides": [4, 2, 1], "noise": True, "depthwise": True}
        import inspect
        accepted = set(inspect.signature(SNAC.__init__).parameters)
        cfg = {k: v for k, v in cfg.items() if k in accepted}
        torch.manual_seed(0)
        snac = SNAC(**cfg)
        snap = _snapshot_dir(cache, SNAC_REPO)
        with open(os.path.join(snap, "config.json"), "w") as f:
            json.dump(cfg, f)
        torch.save(snac.state_dict(), os.path.join(snap, "pytorch_model.bin"))
    finally:
        sys.path.remove(REF)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_reference(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "mstar")):
        return _unavailable("reference is not installed under baseline/_ref")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no GPU visible")
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"torch import failed: {e}")
    work = tempfile.mkdtemp(prefix="mstar_ref_")
    cache = os.path.join(work, "hf")
    proc = None
    log_path = os.path.join(work, "server.log")
    try:
        build_synthetic_cache(cache)
        cfg_path = os.path.join(work, "orpheus_colocated.yaml")
        with open(cfg_path, "w") as f:
            f.write(stock_yaml(args.gpus))
        port = _free_port()
        env = dict(os.environ, PYTHONPATH=REF + os.pathsep + os.environ.get("PYTHONPATH", ""), HF_HUB_OFFLINE="1",
                   TRANSFORMERS_OFFLINE="1", HF_HOME=cache, MASTER_ADDR="127.0.0.1")
        cmd = [sys.executable, "-m", "mstar.api_server.entrypoint", "--config", cfg_path, "--host", "127.0.0.1",
               "--port", str(port), "--tensor-comm-protocol", "SHM", "--cache-dir", cache,
               "--socket-path-prefix", os.path.join(work, "sock"), "--upload-dir", os.path.join(work, "up")]
        logf = open(log_path, "w")
        proc = subprocess.Popen(cmd, env=env, stdout=logf, stderr=subprocess.STDOUT, cwd=work, start_new_session=True)
        import requests
        deadline = time.time() + float(os.environ.get("MSTAR_REF_STARTUP_S", "900"))
        up = False
        while time.time() < deadline and proc.poll() is None:
            try:
                if requests.get(f"http://127.0.0.1:{port}/health", timeout=2).status_code == 200:
                    up = True
                    break
            except Exception:  # noqa: BLE001
                time.sleep(2)
        if not up:
            tail = open(log_path).read()[-600:]
            return _unavailable(f"reference server did not come up (exit {proc.poll()}): {tail}")
        url = f"http://127.0.0.1:{port}/generate"
        sys.path.insert(0, os.path.dirname(HERE))
        from bench import shared_config
        from mstar_b200.bench.tts_client import run_streams, summarize
        C = args.concurrency if hasattr(args, "concurrency") else 64
        N = max(1, args.gpus)
        total = C * N
        W, K = max(3, args.warmup), args.steps
        kw = {"ignore_eos": True, "voice": "tara"}
        # the same warm-up as the other arm: one request, then a short round at full concurrency
        w = run_streams(url, 1, dict(kw, max_output_tokens=28 * 3), text="warm up")
        if w[0]["error"] or not w[0]["chunks"]:
            tail = open(log_path).read()[-600:]
            return _unavailable(f"reference warm-up request failed: {w[0]['error'] or 'no audio'}: {tail}")
        run_streams(url, total, dict(kw, max_output_tokens=56), text="warm {i}")
        # 1204 tokens = 172 audio frames per request
        max_tokens = getattr(args, "gen_tokens", 1204)
        recs = run_streams(url, total, dict(kw, max_output_tokens=max_tokens))
        # bytes per sample from the chunk sizes (16-bit PCM unless the server sends float32)
        sample_bytes = 4 if all(b % 8192 == 0 for r in recs for (_, b) in r["chunks"]) else 2
        try:
            sm = summarize(recs, total, sample_bytes)
        except RuntimeError as e:
            tail = open(log_path).read()[-400:]
            return _unavailable(f"{e} {tail}")
        value = sm["tokens_per_s"]
        return {"metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": N, "steps": K, "warmup": W,
                "ms_per_step": round(1e3 * total / value, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "impl": "reference",
                "data": "synthetic (random-init weights N(0,0.02) in the reference's checkpoint layout, byte tokenizer)",
                "config": dict(shared_config(N, C), placement="reference configs/orpheus_colocated.yaml"
                               + (f" with ranks 0..{N - 1} in both node groups" if N > 1 else ""),
                               timing="wall clock at the HTTP clients over the window in which all requests decode"),
                "ttft_p50_ms": round(sm["ttfa_p50_ms"], 2),
                "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                        "d2h_bytes_per_step": None, "ttfa_p50_ms": round(sm["ttfa_p50_ms"], 2),
                        "ttfa_p99_ms": round(sm["ttfa_p99_ms"], 2)},
                "window_s": round(sm["window_s"], 3)}
    except Exception as e:  # noqa: BLE001
        tail = ""
        try:
            tail = open(log_path).read()[-400:]
        except Exception:  # noqa: BLE001
            pass
        return _unavailable(f"{type(e).__name__}: {e} {tail}")
    finally:
        if proc is not None and proc.poll() is None:
            try:
                os.killpg(proc.pid, 15)          # the launcher's own process group (conductor and workers)
                proc.wait(timeout=20)
            except Exception:  # noqa: BLE001
                try:
                    os.killpg(proc.pid, 9)
                except Exception:  # noqa: BLE001
                    pass
        if os.environ.get("MSTAR_REF_KEEP_LOG"):       # directory to keep the server's log in
            try:
                keep = os.environ["MSTAR_REF_KEEP_LOG"]
                os.makedirs(keep, exist_ok=True)
                shutil.copy(log_path, os.path.join(keep, "reference_server.log"))
            except Exception:  # noqa: BLE001
                pass
        shutil.rmtree(work, ignore_errors=True)
