"""Per-request and aggregate metrics of the benchmark client.

Reference counterparts: ``RequestMetrics`` / ``AggregateMetrics`` / ``LatencyStats`` (benchmark/request.py:30-131,
381-431): TTFT per output modality, inter-token latency, end-to-end latency, audio streaming viability, real-time
factor, request / token / audio-second throughput.
"""
from __future__ import annotations

import statistics
from dataclasses import dataclass, field


@dataclass
class LatencyStats:
    mean: float
    p50: float
    p95: float
    p99: float
    n: int = 0

    @classmethod
    def of(cls, values: list[float]) -> "LatencyStats | None":
        vs = sorted(v for v in values if v is not None)
        if not vs:
            return None

        def pct(p):
            return vs[min(len(vs) - 1, int(round(p / 100 * (len(vs) - 1))))]
        return cls(statistics.mean(vs), pct(50), pct(95), pct(99), len(vs))

    def ms(self) -> str:
        return f"mean {1e3 * self.mean:8.2f}  p50 {1e3 * self.p50:8.2f}  p95 {1e3 * self.p95:8.2f}  p99 {1e3 * self.p99:8.2f} ms"


@dataclass
class RequestMetrics:
    request_id: str
    request_type: str
    t_send: float | None = None                     # time.monotonic() right before the HTTP request leaves
    t_done: float | None = None
    ttft: dict = field(default_factory=dict)        # modality -> seconds to the first chunk of that modality
    arrivals: dict = field(default_factory=dict)    # modality -> [arrival times]
    nbytes: dict = field(default_factory=dict)      # modality -> payload bytes
    units: dict = field(default_factory=dict)       # modality -> tokens (text) / samples (audio) / items
    error: str | None = None
    # audio: (gap to the previous chunk, seconds of audio the previous chunk held) per chunk after the first
    audio_gaps: list = field(default_factory=list)
    _last_audio: tuple | None = None

    def record(self, modality: str, payload_bytes: int, now: float, *, units: int = 1, sample_rate: int = 24000,
               bytes_per_sample: int = 2) -> None:
        self.arrivals.setdefault(modality, []).append(now)
        self.nbytes[modality] = self.nbytes.get(modality, 0) + payload_bytes
        if modality not in self.ttft and self.t_send is not None:
            self.ttft[modality] = now - self.t_send
        if modality == "audio":
            samples = payload_bytes // bytes_per_sample
            self.units["audio"] = self.units.get("audio", 0) + samples
            dur = samples / sample_rate
            if self._last_audio is not None:
                self.audio_gaps.append((now - self._last_audio[0], self._last_audio[1]))
            self._last_audio = (now, dur)
        else:
            self.units[modality] = self.units.get(modality, 0) + units

    @property
    def ok(self) -> bool:
        return self.error is None and self.t_done is not None and bool(self.arrivals)

    @property
    def e2e(self) -> float | None:
        return None if self.t_send is None or self.t_done is None else self.t_done - self.t_send

    def itl(self, modality: str) -> list[float]:
        """Inter-chunk gaps, normalised per unit for text (a chunk may carry several tokens)."""
        ts = self.arrivals.get(modality, [])
        if len(ts) < 2:
            return []
        gaps = [b - a for a, b in zip(ts, ts[1:])]
        if modality == "text" and self.units.get("text", 0) > len(ts):
            per = self.units["text"] / len(ts)
            gaps = [g / per for g in gaps]
        return gaps

    def audio_seconds(self, sample_rate: int = 24000) -> float:
        return self.units.get("audio", 0) / sample_rate

    def streaming_viability(self) -> float | None:
        """Fraction of audio chunks that arrived before the previous chunk finished playing."""
        if not self.audio_gaps:
            return None
        return sum(1 for gap, dur in self.audio_gaps if gap <= dur) / len(self.audio_gaps)


@dataclass
class AggregateMetrics:
    mode: str
    n_requests: int
    n_success: int
    wall_s: float
    ttft: dict            # modality -> LatencyStats
    itl: dict
    e2e: LatencyStats | None
    request_throughput: float
    text_tokens_per_s: float | None = None
    audio_seconds_per_s: float | None = None
    rtf: LatencyStats | None = None                 # per request: end-to-end latency / seconds of audio produced
    streaming_viability: LatencyStats | None = None
    output_bytes: dict = field(default_factory=dict)
    errors: list = field(default_factory=list)
    settings: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        def st(x):
            return None if x is None else dict(mean=x.mean, p50=x.p50, p95=x.p95, p99=x.p99, n=x.n)
        return dict(mode=self.mode, n_requests=self.n_requests, n_success=self.n_success, wall_s=self.wall_s,
                    ttft={k: st(v) for k, v in self.ttft.items()}, itl={k: st(v) for k, v in self.itl.items()},
                    e2e=st(self.e2e), request_throughput=self.request_throughput,
                    text_tokens_per_s=self.text_tokens_per_s, audio_seconds_per_s=self.audio_seconds_per_s,
                    rtf=st(self.rtf), streaming_viability=st(self.streaming_viability), output_bytes=self.output_bytes,
                    errors=self.errors[:10], settings=self.settings)

    def __str__(self) -> str:
        lines = [f"{self.mode} benchmark: {self.n_success}/{self.n_requests} requests ok in {self.wall_s:.2f} s "
                 f"({self.request_throughput:.2f} req/s)", "-" * 78]
        for m, s in sorted(self.ttft.items()):
            lines.append(f"TTFT ({m:<5}) {s.ms()}")
        for m, s in sorted(self.itl.items()):
            lines.append(f"ITL  ({m:<5}) {s.ms()}")
        if self.e2e:
            lines.append(f"E2E          {self.e2e.ms()}")
        if self.text_tokens_per_s:
            lines.append(f"text tokens/s        {self.text_tokens_per_s:10.1f}")
        if self.audio_seconds_per_s:
            lines.append(f"audio seconds/s      {self.audio_seconds_per_s:10.2f}")
        if self.rtf:
            lines.append(f"RTF (latency / audio duration)  mean {self.rtf.mean:.3f}  p50 {self.rtf.p50:.3f}  p95 {self.rtf.p95:.3f}")
        if self.streaming_viability:
            lines.append(f"audio streaming viability       mean {self.streaming_viability.mean:.3f}  p50 {self.streaming_viability.p50:.3f}")
        for e in self.errors[:5]:
            lines.append(f"error: {e}")
        return "\n".join(lines)


def aggregate(metrics: list[RequestMetrics], wall_s: float, mode: str, settings: dict | None = None,
              sample_rate: int = 24000) -> AggregateMetrics:
    ok = [m for m in metrics if m.ok]
    mods = sorted({k for m in ok for k in m.ttft})
    ttft = {k: LatencyStats.of([m.ttft.get(k) for m in ok]) for k in mods}
    itl = {k: LatencyStats.of([g for m in ok for g in m.itl(k)]) for k in mods}
    text_tokens = sum(m.units.get("text", 0) for m in ok)
    audio_s = sum(m.audio_seconds(sample_rate) for m in ok)
    rtf = LatencyStats.of([m.e2e / m.audio_seconds(sample_rate) for m in ok if m.audio_seconds(sample_rate) > 0])
    sv = LatencyStats.of([m.streaming_viability() for m in ok])
    nbytes: dict = {}
    for m in ok:
        for k, v in m.nbytes.items():
            nbytes[k] = nbytes.get(k, 0) + v
    return AggregateMetrics(mode, len(metrics), len(ok), wall_s, {k: v for k, v in ttft.items() if v},
                            {k: v for k, v in itl.items() if v}, LatencyStats.of([m.e2e for m in ok]),
                            len(ok) / wall_s if wall_s > 0 else 0.0,
                            text_tokens / wall_s if text_tokens and wall_s > 0 else None,
                            audio_s / wall_s if audio_s and wall_s > 0 else None, rtf, sv, nbytes,
                            [m.error for m in metrics if m.error], settings or {})
