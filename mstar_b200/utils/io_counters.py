"""Process-wide byte counters of host <-> device copies made by the serving path (plan uploads, token and waveform
read-backs, status words), so that a benchmark can report the bytes per step from the tensors actually copied."""
from __future__ import annotations

h2d_bytes = 0
d2h_bytes = 0


def add_h2d(n: int) -> None:
    global h2d_bytes
    h2d_bytes += int(n)


def add_d2h(n: int) -> None:
    global d2h_bytes
    d2h_bytes += int(n)


def snapshot() -> dict:
    return {"h2d_bytes": h2d_bytes, "d2h_bytes": d2h_bytes}
