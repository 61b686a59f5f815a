"""Rendering of a request profile as the tree that ``--log-stats`` prints when a request completes.

Reference counterpart: ``pretty_print_profile`` (mstar/profile/display.py:29-167)."""
from __future__ import annotations

from .records import RequestProfile

_ORDER = ["received", "preprocessed", "admitted", "first_chunk", "last_chunk", "conductor_done", "finished"]


def _bytes(n: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB"):
        if n < 1024 or unit == "GiB":
            return f"{n:.0f} {unit}" if unit == "B" else f"{n:.1f} {unit}"
        n /= 1024
    return f"{n:.1f} GiB"


def _ms(s: float) -> str:
    return f"{1e3 * s:9.2f} ms"


def render(prof: RequestProfile) -> str:
    out = [f"request {prof.request_id}"]
    if prof.inputs or prof.outputs:
        out.append("├─ data")
        for label, d in (("in ", prof.inputs), ("out", prof.outputs)):
            for mod, (cnt, nb) in sorted(d.items()):
                out.append(f"│    {label} {mod:<8} x{cnt:<5} {_bytes(nb):>10}")
    cps = sorted(((k, v) for k, v in prof.checkpoints.items() if v is not None),
                 key=lambda kv: (kv[1], _ORDER.index(kv[0]) if kv[0] in _ORDER else 99))
    if len(cps) >= 2:
        out.append("├─ timeline")
        for (a, ta), (b, tb) in zip(cps, cps[1:]):
            out.append(f"│    {a + ' -> ' + b:<34} {_ms(tb - ta)}")
        out.append(f"│    {'total':<34} {_ms(cps[-1][1] - cps[0][1])}   tokens out {prof.tokens_out}")
    if prof.nodes:
        out.append("├─ nodes: executions (iterations, mean batch) | launch | in flight | post, totals (mean per execution)")
        last = None
        for nt in sorted(prof.nodes, key=lambda x: (x.worker, x.node, x.walk)):
            if (nt.worker, nt.node) != last:
                out.append(f"│    {nt.node} @ {nt.worker}")
                last = (nt.worker, nt.node)
            n = max(1, nt.executions)
            spec = f", {nt.speculative} speculative" if nt.speculative else ""
            out.append(f"│      {nt.walk:<18} x{nt.executions} ({nt.iterations} it, batch {nt.batch_rows / n:.1f}{spec})")
            out.append(f"│        launch {_ms(nt.launch_s)} ({_ms(nt.launch_s / n).strip()})   in flight {_ms(nt.flight_s)} "
                       f"({_ms(nt.flight_s / n).strip()})   post {_ms(nt.post_s)} ({_ms(nt.post_s / n).strip()})")
        out.append("│      in-flight times of speculative executions overlap: they do not add up to wall time")
    if prof.transfers:
        out.append("└─ tensor transfers between processes")
        for tr in sorted(prof.transfers, key=lambda t: (t.direction, t.src, t.dst, t.edge)):
            arrow = f"{tr.src} -> {tr.dst}"
            out.append(f"     {tr.direction} {arrow:<28} {tr.edge:<18} x{tr.count:<5} {_bytes(tr.nbytes):>10} {_ms(tr.seconds)}")
    else:
        out[-1] = out[-1].replace("│", " ", 1) if out[-1].startswith("│") else out[-1]
    return "\n".join(out)


def format_profile(request_id: str, prof: dict, t_submit: float | None = None, t_first: float | None = None) -> str:
    """Render the profile dictionary that ``REQUEST_COMPLETE`` carries (tolerates the bare conductor summary)."""
    rp = RequestProfile.from_dict(dict(prof.get("request", {}), request_id=request_id)) if "request" in prof \
        else RequestProfile(request_id)
    if not rp.checkpoints:
        rp.checkpoints = {"received": 0.0, "admitted": prof.get("queue_s", 0.0), "finished": prof.get("total_s", 0.0)}
        if t_submit is not None and t_first is not None:
            rp.checkpoints["first_chunk"] = t_first - t_submit
    rp.tokens_out = rp.tokens_out or int(prof.get("tokens_out", 0))
    for w in prof.get("walks", []):
        if isinstance(w, dict) and w.get("profile"):
            rp.merge_worker(w["profile"])
    return render(rp)


def write_profile(text: str, filename: str | None = None) -> None:
    if filename:
        with open(filename, "a") as f:
            f.write(text + "\n")
    else:
        print(text, flush=True)
