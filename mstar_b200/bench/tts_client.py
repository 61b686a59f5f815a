"""Load generator for the streaming TTS benchmark: N concurrent ``POST /generate`` requests (NDJSON reply), the
arrival time and size of every audio chunk recorded at the client. Both arms of ``bench.py`` (this framework's
server and the reference's) are driven by this same client, so client cost is identical on both sides.

The streams are spread over several client PROCESSES (asyncio + aiohttp inside each): hundreds of streams at tens of
thousands of tokens per second would otherwise be limited by one interpreter's lock rather than by the server.
Times are ``time.monotonic()``, which is one clock for all processes of a machine.

    python -m mstar_b200.bench.tts_client --url http://127.0.0.1:8000/generate --n 64 --kwargs '{"max_tokens": 84}'
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import time


async def _one(session, url: str, text: str, kwargs: dict, start_at: float) -> dict:
    rec = {"t_submit": None, "t_first": None, "t_done": None, "chunks": [], "error": None}
    await asyncio.sleep(max(0.0, start_at - time.monotonic()))
    try:
        rec["t_submit"] = time.monotonic()
        data = {"text": text, "output_modalities": "audio", "streaming": "true", "model_kwargs": json.dumps(kwargs)}
        async with session.post(url, data=data) as resp:
            if resp.status != 200:
                rec["error"] = f"HTTP {resp.status}: {(await resp.text())[:200]}"
            else:
                async for line in resp.content:
                    if len(line) < 8:
                        continue
                    try:
                        msg = json.loads(line)
                    except Exception:  # noqa: BLE001
                        continue
                    mod = msg.get("modality")
                    payload = msg.get("data") or ""
                    if mod == "error":
                        import base64
                        rec["error"] = base64.b64decode(payload).decode(errors="replace")[:300]
                        break
                    if mod == "audio" and payload:
                        n = (len(payload) * 3) // 4 - payload.count("=", -2)
                        now = time.monotonic()
                        if rec["t_first"] is None:
                            rec["t_first"] = now
                        rec["chunks"].append((now, n))
    except Exception as e:  # noqa: BLE001
        rec["error"] = f"{type(e).__name__}: {e}"
    rec["t_done"] = time.monotonic()
    return rec


async def _many(url: str, n: int, first: int, kwargs: dict, start_at: float, text: str) -> list[dict]:
    import aiohttp
    timeout = aiohttp.ClientTimeout(total=3600)
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(timeout=timeout, connector=conn, read_bufsize=1 << 21) as session:
        return await asyncio.gather(*[_one(session, url, text.format(i=first + i), kwargs, start_at)
                                      for i in range(n)])


def run_streams(url: str, n: int, kwargs: dict, *, per_process: int = 32, text: str = "request number {i} says hello",
                timeout_s: float = 3600.0) -> list[dict]:
    """Run ``n`` concurrent streams (all submitted at the same instant) and return one record per stream:
    ``t_submit``, ``t_first`` (first audio chunk), ``t_done``, ``chunks`` [(time, audio bytes)], ``error``."""
    start_at = time.monotonic() + 1.5 + 0.002 * n          # interpreter start-up of the client processes
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs, first = [], 0
    while first < n:
        k = min(per_process, n - first)
        procs.append(subprocess.Popen([sys.executable, "-m", "mstar_b200.bench.tts_client", "--url", url, "--n", str(k),
                                       "--first", str(first), "--kwargs", json.dumps(kwargs), "--start-at",
                                       repr(start_at), "--text", text], stdout=subprocess.PIPE, text=True,
                                      env=env, cwd=root))
        first += k
    recs: list[dict] = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout_s)
            recs.extend(json.loads(out.strip().splitlines()[-1]))
        except Exception as e:  # noqa: BLE001
            p.kill()
            recs.append({"t_submit": None, "t_first": None, "t_done": time.monotonic(), "chunks": [],
                         "error": f"client process failed: {type(e).__name__}: {e}"})
    return recs


def summarize(recs: list[dict], concurrency: int, sample_bytes: int = 2) -> dict:
    """Tokens per second over the window in which every stream decodes (opens when the last stream has delivered its
    first audio, closes when the first stream ends; 7 tokens per 2048 samples), and time to first audio."""
    import statistics
    bad = [r["error"] for r in recs if r["error"] or not r["chunks"]]
    if bad:
        raise RuntimeError(f"{len(bad)} of {len(recs)} requests failed: {bad[0]}")
    t_open, t_close = max(r["t_first"] for r in recs), min(r["t_done"] for r in recs)
    if t_close <= t_open:
        raise RuntimeError("measurement window is empty (requests did not overlap)")
    nbytes = sum(b for r in recs for (t, b) in r["chunks"] if t_open < t <= t_close)
    tokens = nbytes / sample_bytes / 2048 * 7
    dt = t_close - t_open
    ttfa = [(r["t_first"] - r["t_submit"]) * 1e3 for r in recs]
    total_bytes = sum(b for r in recs for (_, b) in r["chunks"])
    return {"tokens_per_s": tokens / dt, "window_s": dt, "ttfa_p50_ms": statistics.median(ttfa),
            "ttfa_p99_ms": sorted(ttfa)[min(len(ttfa) - 1, int(0.99 * len(ttfa)))],
            "ms_per_step": 1e3 * concurrency * dt / max(tokens, 1.0),
            "audio_tokens_total": total_bytes / sample_bytes / 2048 * 7,
            "wall_s": max(r["t_done"] for r in recs) - min(r["t_submit"] for r in recs)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", required=True)
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--first", type=int, default=0)
    ap.add_argument("--kwargs", default="{}")
    ap.add_argument("--start-at", type=float, default=0.0)
    ap.add_argument("--text", default="request number {i} says hello")
    a = ap.parse_args()
    recs = asyncio.run(_many(a.url, a.n, a.first, json.loads(a.kwargs), a.start_at, a.text))
    print(json.dumps(recs))


if __name__ == "__main__":
    main()
