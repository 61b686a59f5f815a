"""Benchmark runner: fires requests at a running server and reports latency and throughput metrics.

Firing modes: ``offline`` (batches of ``--batch-size`` sent together, next batch when the last one is done),
``closed_loop`` (``--max-concurrency`` requests in flight at all times) and ``online`` (Poisson arrivals at
``--rate`` requests per second).

Reference counterparts: ``BenchmarkRunner`` (benchmark/runner.py:127-490: _run_batch, _run_concurrent_offline /
_online / _closed_loop, _warmup, _write_results_json) and its command line (:492-688).
"""
from __future__ import annotations

import argparse
import asyncio
import base64
import json
import random
import time

from .metrics import AggregateMetrics, RequestMetrics, aggregate
from .requests import REQUEST_TYPES, RequestInput, make_requests


async def send_request(session, url: str, req: RequestInput, rid: str, sample_rate: int = 24000) -> RequestMetrics:
    import aiohttp
    m = RequestMetrics(rid, req.request_type)
    data, files = req.form()
    form = aiohttp.FormData()
    for k, v in data.items():
        form.add_field(k, v)
    form.add_field("request_id", rid)
    for name, blob in files:
        form.add_field("files", blob, filename=name)
    try:
        m.t_send = time.monotonic()
        async with session.post(url + "/generate", data=form) as resp:
            if resp.status != 200:
                m.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
            else:
                async for line in resp.content:
                    if len(line) < 8:
                        continue
                    msg = json.loads(line)
                    mod, payload = msg.get("modality"), msg.get("data") or ""
                    now = time.monotonic()
                    if mod == "error":
                        m.error = base64.b64decode(payload).decode(errors="replace")[:300]
                        break
                    n = (len(payload) * 3) // 4 - payload.count("=", -2)
                    units = 1
                    if mod == "text":       # one chunk may carry several space-separated tokens
                        units = max(1, len(base64.b64decode(payload).split()))
                    m.record(mod, n, now, units=units, sample_rate=sample_rate)
    except Exception as e:  # noqa: BLE001
        m.error = f"{type(e).__name__}: {e}"
    m.t_done = time.monotonic()
    return m


class BenchmarkRunner:
    def __init__(self, url: str, requests: list[RequestInput], *, mode: str = "closed_loop", batch_size: int = 1,
                 max_concurrency: int = 8, rate: float = 1.0, warmup: int = 1, seed: int = 0, sample_rate: int = 24000):
        self.url, self.requests, self.mode = url.rstrip("/"), requests, mode
        self.batch_size, self.max_concurrency, self.rate = batch_size, max_concurrency, rate
        self.warmup, self.seed, self.sample_rate = warmup, seed, sample_rate

    async def _one(self, session, i: int, req: RequestInput, tag: str = "bench") -> RequestMetrics:
        return await send_request(session, self.url, req, f"{tag}-{i}-{random.getrandbits(32):08x}", self.sample_rate)

    async def _offline(self, session) -> list[RequestMetrics]:
        out = []
        for s in range(0, len(self.requests), self.batch_size):
            out += await asyncio.gather(*[self._one(session, s + j, r)
                                          for j, r in enumerate(self.requests[s:s + self.batch_size])])
        return out

    async def _closed_loop(self, session) -> list[RequestMetrics]:
        sem = asyncio.Semaphore(self.max_concurrency)

        async def limited(i, r):
            async with sem:
                return await self._one(session, i, r)
        return await asyncio.gather(*[limited(i, r) for i, r in enumerate(self.requests)])

    async def _online(self, session) -> list[RequestMetrics]:
        rng = random.Random(self.seed)
        tasks = []
        for i, r in enumerate(self.requests):
            tasks.append(asyncio.ensure_future(self._one(session, i, r)))
            await asyncio.sleep(rng.expovariate(self.rate))
        return await asyncio.gather(*tasks)

    async def run(self) -> tuple[list[RequestMetrics], AggregateMetrics]:
        import aiohttp
        timeout = aiohttp.ClientTimeout(total=3600)
        async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0),
                                         read_bufsize=1 << 22) as session:
            for i, r in enumerate(self.requests[:self.warmup]):
                w = await self._one(session, i, r, tag="warmup")
                if w.error:
                    raise RuntimeError(f"warm-up request failed: {w.error}")
            t0 = time.monotonic()
            ms = await {"offline": self._offline, "closed_loop": self._closed_loop, "online": self._online}[self.mode](session)
            wall = time.monotonic() - t0
        settings = dict(url=self.url, mode=self.mode, batch_size=self.batch_size, max_concurrency=self.max_concurrency,
                        rate=self.rate, warmup=self.warmup, request_type=self.requests[0].request_type if self.requests else "")
        return ms, aggregate(ms, wall, self.mode, settings, self.sample_rate)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="mstar-bench")
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--request-type", default="t2t", choices=sorted(REQUEST_TYPES))
    ap.add_argument("--num-requests", type=int, default=16)
    ap.add_argument("--num-warmup", type=int, default=1)
    ap.add_argument("--mode", default="closed_loop", choices=["offline", "closed_loop", "online"])
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--max-concurrency", type=int, default=8)
    ap.add_argument("--rate", type=float, default=1.0, help="requests per second (online mode)")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--audio-seconds", type=float, default=5.0)
    ap.add_argument("--numeric-prompts", action="store_true", help="prompts as token ids (server without a tokenizer)")
    ap.add_argument("--model-kwargs", default="{}", help="JSON merged into every request's model_kwargs")
    ap.add_argument("--sample-rate", type=int, default=24000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json", default=None, help="write the aggregate and per-request metrics here")
    a = ap.parse_args(argv)
    reqs = make_requests(a.request_type, a.num_requests, seed=a.seed, max_tokens=a.max_tokens, image_size=a.image_size,
                         audio_seconds=a.audio_seconds, extra_kwargs=json.loads(a.model_kwargs),
                         numeric_prompts=a.numeric_prompts)
    runner = BenchmarkRunner(a.url, reqs, mode=a.mode, batch_size=a.batch_size, max_concurrency=a.max_concurrency,
                             rate=a.rate, warmup=a.num_warmup, seed=a.seed, sample_rate=a.sample_rate)
    ms, agg = asyncio.run(runner.run())
    print(agg)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"aggregate": agg.to_dict(),
                       "requests": [dict(request_id=m.request_id, ttft=m.ttft, e2e=m.e2e, nbytes=m.nbytes, units=m.units,
                                         error=m.error, streaming_viability=m.streaming_viability()) for m in ms]}, f)


if __name__ == "__main__":
    main()
