"""Per-request timing report (``--log-stats``). Reference counterparts: mstar/profile/format.py,
mstar/profile/display.py:29-167."""
from __future__ import annotations


def format_profile(request_id: str, prof: dict, t_submit: float, t_first: float | None) -> str:
    lines = [f"request {request_id}:"]
    if t_first is not None:
        lines.append(f"  time to first chunk  {1e3 * (t_first - t_submit):9.2f} ms")
    lines.append(f"  queueing             {1e3 * prof.get('queue_s', 0.0):9.2f} ms")
    lines.append(f"  total                {1e3 * prof.get('total_s', 0.0):9.2f} ms   tokens out {prof.get('tokens_out', 0)}")
    for w in prof.get("walks", []):
        lines.append(f"    walk {w.get('walk', '?'):<18} {1e3 * w.get('walk_s', 0.0):9.2f} ms")
    return "\n".join(lines)
