"""Command line: ``mstar serve <model-or-config>`` starts the server; ``mstar build`` compiles the native
libraries. Reference counterparts: mstar/cli/main.py:25-209 and the ``mstar-serve`` flags
(mstar/api_server/entrypoint.py:830-993)."""
from __future__ import annotations

import argparse
import logging
import os
import sys
from pathlib import Path

CONFIG_DIR = Path(__file__).resolve().parents[2] / "configs"
DEFAULT_CONFIGS = {
    "tiny": "tiny.yaml", "orpheus": "orpheus.yaml", "bagel": "bagel.yaml", "qwen3_omni": "qwen3omni.yaml",
    "qwen3omni": "qwen3omni.yaml", "cosmos3": "cosmos3_nano.yaml", "wan22": "wan22.yaml", "pi05": "pi05.yaml",
    "vjepa2": "vjepa2.yaml", "qwen3_tts": "qwen3tts.yaml", "whisper_large": "whisper_large.yaml",
    "higgs_audio": "higgs_audio.yaml",
}


def resolve_config(model_or_path: str) -> str:
    if os.path.exists(model_or_path):
        return model_or_path
    name = DEFAULT_CONFIGS.get(model_or_path, model_or_path + ".yaml")
    p = CONFIG_DIR / name
    if not p.exists():
        raise SystemExit(f"no config for {model_or_path!r} (looked for {p})")
    return str(p)


def add_serve_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--config", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--timeout", type=float, default=float(os.environ.get("MSTAR_REQUEST_TIMEOUT_S", 600)))
    ap.add_argument("--enable-nvtx", action="store_true")
    ap.add_argument("--log-level", default="INFO")
    ap.add_argument("--log-stats", action="store_true", help="print a per-request profile when a request completes")
    ap.add_argument("--log-stats-file", default=None, help="append the per-request profiles to this file instead")
    ap.add_argument("--multi-process", action="store_true", help="one OS process per worker over the shm mesh")
    ap.add_argument("--native-frontend", action="store_true", help="serve HTTP from the C++ frontend (mstar-server)")
    ap.add_argument("--cache-dir", default=None)
    ap.add_argument("--allow-remote-media", action="store_true")


def serve(args) -> None:
    logging.basicConfig(level=args.log_level)
    from ..api_server.app import create_app
    from ..api_server.server import APIServer
    from ..utils import profiler
    profiler.enable(args.enable_nvtx)
    cfg = args.config or resolve_config(args.model)
    server = APIServer(cfg, in_process=not args.multi_process, request_timeout_s=args.timeout,
                       log_stats=args.log_stats, log_stats_file=args.log_stats_file).start()
    if args.native_frontend:
        from ..api_server.native_frontend import NativeFrontend
        fe = NativeFrontend(create_app(server, args.allow_remote_media), host=args.host, port=args.port).start()
        try:
            fe.wait()
        finally:
            fe.stop()
            server.shutdown()
        return
    import uvicorn
    try:
        uvicorn.run(create_app(server, args.allow_remote_media), host=args.host, port=args.port, log_level=args.log_level.lower())
    finally:
        server.shutdown()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="mstar")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="start the server")
    s.add_argument("model", nargs="?", default="tiny")
    add_serve_flags(s)
    sub.add_parser("build", help="compile the native libraries for sm_100a")
    args = ap.parse_args(argv)
    if args.cmd == "build":
        from .. import build
        build.build_all(verbose=True)
    else:
        serve(args)


def serve_main(argv=None) -> None:
    """``mstar-serve --config <yaml>``"""
    ap = argparse.ArgumentParser(prog="mstar-serve")
    add_serve_flags(ap)
    args = ap.parse_args(argv)
    args.model = "tiny"
    if not args.config:
        raise SystemExit("--config is required")
    serve(args)


if __name__ == "__main__":
    main()
